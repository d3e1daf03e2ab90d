// Host-side check of comet_b200/csrc/mtxparse.cuh (the line parser the device kernels run): every
// line it accepts must give exactly what strtoll / strtod give.  Prints "ok <accepted> <sent to host>".
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <random>
#include <string>

#include "../../comet_b200/csrc/mtxparse.cuh"

using namespace cb200;

static int check_double(const std::string &s, long *ok, long *host)
{
    double got = 0;
    const char *next = nullptr;
    const int st = mtx_parse_double(s.data(), s.data() + s.size(), &got, &next);
    char *endp = nullptr;
    const double want = strtod(s.c_str(), &endp);
    if (st == PARSE_OK) {
        if (memcmp(&got, &want, 8) != 0 || next != s.data() + (endp - s.c_str())) {
            printf("MISMATCH '%s': got %.17g (%a) want %.17g (%a) consumed %ld vs %ld\n", s.c_str(), got, got, want, want,
                   (long)(next - s.data()), (long)(endp - s.c_str()));
            return 1;
        }
        (*ok)++;
    } else if (st == PARSE_HOST) {
        (*host)++;
    } else if (endp != s.c_str()) {
        printf("REFUSED '%s' although strtod converts it\n", s.c_str());
        return 1;
    }
    return 0;
}

int main(int argc, char **argv)
{
    const long n = argc > 1 ? atol(argv[1]) : 200000;
    std::mt19937_64 rng(12345);
    long ok = 0, host = 0;
    char buf[128];
    const char *fixed[] = {"0", "-0", "0.0", "1", "1.0", "-1.5", "2.5e0", "1e0", "1E5", "1e-5", ".5", "5.", "+3.25", "1e19", "1e20",
                           "9007199254740993", "9007199254740992.5", "0.1", "0.2", "0.30000000000000004", "123456789012345678",
                           "1234567890123456789", "12345678901234567890", "1e-38", "1e-39", "4.9e-324", "1.7976931348623157e308",
                           "1e400", "0.000000000000000000000000000000000000001", "1e", "1e+", "1.5x", "inf", "nan", "-inf", "0x10",
                           "  7.25", "\t-8.125e-3 trailing", "0.5 0.25", "5e-1", "1.0000000000000002", "1.00000000000000011102230246251565404",
                           "2.2250738585072014e-308", "2.2250738585072011e-308", "8.5", "00012.5", "-.75e1", "", "abc", ".", "-", "+.e1"};
    for (const char *f : fixed)
        if (check_double(f, &ok, &host)) return 1;
    for (long i = 0; i < n; i++) {
        const int kind = (int)(rng() % 6);
        std::string s;
        if (kind == 0) {                       // what the benchmark writes: %.17g of U(-1, 1) and of U(0.5, 1.5)
            const double u = (double)(rng() >> 11) * (1.0 / 9007199254740992.0);
            snprintf(buf, sizeof(buf), "%.17g", (i & 1) ? 2 * u - 1 : u + 0.5);
            s = buf;
        } else if (kind == 1) {                // shortest-looking decimals
            snprintf(buf, sizeof(buf), "%.*g", 1 + (int)(rng() % 17), ldexp((double)(rng() >> 11), (int)(rng() % 120) - 90));
            s = buf;
        } else if (kind == 2) {                // random digit strings with a point somewhere
            int nd = 1 + (int)(rng() % 22), pt = (int)(rng() % (nd + 1));
            if (rng() % 3 == 0) s += "-";
            for (int d = 0; d < nd; d++) { if (d == pt) s += "."; s += (char)('0' + rng() % 10); }
        } else if (kind == 3) {                // exponents across and beyond the exact range
            snprintf(buf, sizeof(buf), "%llue%d", (unsigned long long)(rng() % 1000000000000000000ull), (int)(rng() % 90) - 50);
            s = buf;
        } else if (kind == 4) {                // halfway cases: 2^53 + odd, and decimal expansions of midpoints
            const unsigned long long b = 9007199254740992ull + (rng() % 4096);
            snprintf(buf, sizeof(buf), "%llu.%s", b, (rng() & 1) ? "5" : "50000000000000000001");
            s = buf;
        } else {
            const double v = ldexp(1.0 + (double)(rng() >> 12) / 4503599627370496.0, (int)(rng() % 60) - 40);
            snprintf(buf, sizeof(buf), "%.*e", 16 + (int)(rng() % 4), v);   // 17..20 significant digits
            s = buf;
        }
        if (check_double(s, &ok, &host)) return 1;
    }
    // integers and whole lines
    const char *lines[] = {"3 4 1.5", "  12\t7   -2.5e-3", "5 6", "1 1 0", "010 2 1.0", "0x1 2 3", "7", "a b c", "3 -4 2", "99999999999999999999 1 1"};
    for (const char *l : lines) {
        int64_t r = -7, c = -7;
        double v = -7;
        const int st = mtx_parse_entry(l, l + strlen(l), false, &r, &c, &v);
        char *t1, *t2, *t3;
        const long long wr = strtoll(l, &t1, 0), wc = strtoll(t1, &t2, 0);
        double wv = strtod(t2, &t3);
        if (t3 == t2) wv = 1.0;
        const bool ref_ok = t1 != l && t2 != t1;
        if (st == PARSE_OK && (!ref_ok || r != wr || c != wc || memcmp(&v, &wv, 8) != 0)) {
            printf("LINE MISMATCH '%s'\n", l);
            return 1;
        }
        if (st == PARSE_BAD && ref_ok) { printf("LINE REFUSED '%s'\n", l); return 1; }
    }
    printf("ok %ld %ld\n", ok, host);
    return 0;
}
