// Parsing one entry line of a MatrixMarket file: "row col [value]" (coordinate files) or "value"
// (array files).  Written to run on the device, one thread per line, and compiled for the host too, so
// that the same code can be checked against strtoll / strtod on a CPU.
//
// The reference reader parses with strtoll(.., 0) and strtod (lib/ExecutionEngine/SparseUtils.cpp
// :145-356), so a value must come out as the CORRECTLY ROUNDED double of the decimal text, bit for bit.
// That is done exactly, without tables: up to 19 significant digits are collected into a 64-bit integer M
// and the value M * 10^e is formed with 128-bit integer arithmetic --
//   e >= 0 : M * 10^e as an exact 128-bit integer (e <= 19),
//   e <  0 : the first 64 significant bits of M / 10^-e by shift-and-subtract long division
//            (10^-e < 2^127, i.e. e >= -38), with a sticky flag for a non-zero remainder --
// and rounded once to 53 bits, ties to even.  Anything outside what this covers exactly (more than 19
// significant digits, exponents beyond the ranges above, results outside the normal doubles, hexadecimal
// or octal integers, inf / nan) is reported as PARSE_HOST: the caller re-parses that line on the host with
// strtoll / strtod, so the result is the reference's in every case.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define MTX_HD __host__ __device__ __forceinline__
#else
#define MTX_HD static inline
#endif

namespace cb200 {

enum { PARSE_OK = 0, PARSE_HOST = 1, PARSE_BAD = 2 };

typedef unsigned __int128 mtx_u128;

MTX_HD bool mtx_space(char ch)
{
    return ch == ' ' || ch == '\t' || ch == '\r' || ch == '\v' || ch == '\f';
}

MTX_HD int mtx_msb(mtx_u128 v)     // position of the highest set bit, v != 0
{
    const uint64_t hi = (uint64_t)(v >> 64), lo = (uint64_t)v;
    int n = 0;
    uint64_t x = hi ? hi : lo;
    while (x >>= 1) n++;
    return hi ? n + 64 : n;
}

// v * 2^exp2 (sticky: the true value lies strictly above v * 2^exp2 by less than one unit of v) rounded to
// double, ties to even.  False when the result is not a normal double.
MTX_HD bool mtx_round_to_double(mtx_u128 v, int exp2, bool sticky, bool negative, double *out)
{
    if (v == 0) {
        if (sticky) return false;
        *out = negative ? -0.0 : 0.0;
        return true;
    }
    const int msb = mtx_msb(v);
    uint64_t mant;
    int e = exp2 + msb;                                 // value in [2^e, 2^(e+1))
    if (msb > 52) {
        const int shift = msb - 52;
        mant = (uint64_t)(v >> shift);
        const mtx_u128 rem = v & ((((mtx_u128)1) << shift) - 1);
        const mtx_u128 half = ((mtx_u128)1) << (shift - 1);
        if (rem > half || (rem == half && (sticky || (mant & 1)))) mant++;
        if (mant >> 53) { mant >>= 1; e++; }
    } else {
        mant = (uint64_t)v << (52 - msb);               // exact (sticky bits lie below the 53rd bit only if msb > 52...
        if (sticky) return false;                       // ...so with fewer than 53 bits and a remainder we do not decide here)
    }
    if (e < -1022 || e > 1023) return false;
    const uint64_t bits = ((uint64_t)negative << 63) | ((uint64_t)(e + 1023) << 52) | (mant & ((1ull << 52) - 1));
    union { uint64_t u; double d; } cv;
    cv.u = bits;
    *out = cv.d;
    return true;
}

MTX_HD mtx_u128 mtx_pow10(int k)    // 10^k, k <= 38
{
    mtx_u128 p = 1;
    for (int i = 0; i < k; i++) p *= 10;
    return p;
}

// Decimal floating-point text at [p, end) -> double.  *next receives the first character not consumed.
// PARSE_BAD: no number here (strtod would convert nothing).
MTX_HD int mtx_parse_double(const char *p, const char *end, double *out, const char **next)
{
    while (p < end && mtx_space(*p)) p++;
    const char *start = p;
    bool negative = false;
    if (p < end && (*p == '+' || *p == '-')) { negative = *p == '-'; p++; }
    if (p >= end) { *next = start; return PARSE_BAD; }
    if (!((*p >= '0' && *p <= '9') || *p == '.')) {
        // inf, nan or junk: strtod decides
        const char ch = *p | 0x20;
        *next = start;
        return (ch == 'i' || ch == 'n') ? PARSE_HOST : PARSE_BAD;
    }
    if (*p == '0' && p + 1 < end && ((p[1] | 0x20) == 'x')) { *next = start; return PARSE_HOST; }   // hexadecimal float
    uint64_t m = 0;
    int sig = 0, exp10 = 0, ndigits = 0;
    bool inexact = false;
    for (; p < end && *p >= '0' && *p <= '9'; p++) {
        ndigits++;
        if (sig == 0 && *p == '0') continue;            // leading zeros
        if (sig < 19) { m = m * 10 + (uint64_t)(*p - '0'); sig++; }
        else { exp10++; if (*p != '0') inexact = true; }
    }
    if (p < end && *p == '.') {
        p++;
        for (; p < end && *p >= '0' && *p <= '9'; p++) {
            ndigits++;
            if (sig == 0 && *p == '0') { exp10--; continue; }
            if (sig < 19) { m = m * 10 + (uint64_t)(*p - '0'); sig++; exp10--; }
            else if (*p != '0') inexact = true;
        }
    }
    if (ndigits == 0) { *next = start; return PARSE_BAD; }
    if (p < end && (*p | 0x20) == 'e') {
        const char *q = p + 1;
        bool eneg = false;
        if (q < end && (*q == '+' || *q == '-')) { eneg = *q == '-'; q++; }
        if (q < end && *q >= '0' && *q <= '9') {
            int ex = 0;
            for (; q < end && *q >= '0' && *q <= '9'; q++)
                if (ex < 100000) ex = ex * 10 + (*q - '0');
            exp10 += eneg ? -ex : ex;
            p = q;
        }
    }
    *next = p;
    if (inexact) return PARSE_HOST;
    if (m == 0) { *out = negative ? -0.0 : 0.0; return PARSE_OK; }
    if (exp10 >= 0) {
        if (exp10 > 19) return PARSE_HOST;
        return mtx_round_to_double((mtx_u128)m * mtx_pow10(exp10), 0, false, negative, out) ? PARSE_OK : PARSE_HOST;
    }
    const int k = -exp10;
    if (k > 38) return PARSE_HOST;
    const mtx_u128 d = mtx_pow10(k);
    // m / d: integer part, then one quotient bit per step until 64 significant bits are there
    mtx_u128 rem = (mtx_u128)m;
    uint64_t q = (uint64_t)(rem / d);
    rem = rem % d;
    int t = 0;
    while (!(q >> 63)) {
        if (rem == 0 && q != 0) break;                  // exact: no need for more bits
        rem <<= 1;
        q <<= 1;
        t++;
        if (rem >= d) { rem -= d; q |= 1; }
        if (t > 260) return PARSE_HOST;
    }
    return mtx_round_to_double((mtx_u128)q, -t, rem != 0, negative, out) ? PARSE_OK : PARSE_HOST;
}

// Decimal integer as strtoll(.., 0) reads it; anything that strtoll would read in another base goes to the host.
MTX_HD int mtx_parse_int(const char *p, const char *end, int64_t *out, const char **next)
{
    while (p < end && mtx_space(*p)) p++;
    const char *start = p;
    bool negative = false;
    if (p < end && (*p == '+' || *p == '-')) { negative = *p == '-'; p++; }
    if (p >= end || *p < '0' || *p > '9') { *next = start; return PARSE_BAD; }
    if (*p == '0' && p + 1 < end && ((p[1] >= '0' && p[1] <= '9') || (p[1] | 0x20) == 'x')) { *next = start; return PARSE_HOST; }
    uint64_t v = 0;
    int nd = 0;
    for (; p < end && *p >= '0' && *p <= '9'; p++) {
        if (++nd > 18) { *next = start; return PARSE_HOST; }
        v = v * 10 + (uint64_t)(*p - '0');
    }
    *out = negative ? -(int64_t)v : (int64_t)v;
    *next = p;
    return PARSE_OK;
}

// One entry line [p, end) (no newline inside).  Coordinate files: 1-based row and column, optional value
// (1.0 when absent).  Array files: the value only.
MTX_HD int mtx_parse_entry(const char *p, const char *end, bool array, int64_t *row, int64_t *col, double *val)
{
    const char *t = p;
    if (array) {
        const int s = mtx_parse_double(p, end, val, &t);
        if (s == PARSE_BAD) { *val = 0.0; return PARSE_OK; }   // strtod converting nothing yields 0.0
        return s;
    }
    int s = mtx_parse_int(p, end, row, &t);
    if (s != PARSE_OK) return s;
    s = mtx_parse_int(t, end, col, &t);
    if (s != PARSE_OK) return s;
    s = mtx_parse_double(t, end, val, &t);
    if (s == PARSE_BAD) { *val = 1.0; return PARSE_OK; }       // pattern entry
    return s;
}

}  // namespace cb200
