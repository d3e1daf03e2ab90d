# lit settings of the libcomet_b200 tests (a COMET checkout with integration/comet/ copied over it).
# They need a B200 and the library: configure with -DCOMET_B200_LIBRARY=<path>/libcomet_b200.so, which
# sets config.comet_b200_library; without it the tests are unsupported rather than failed.
config.suffixes = ['.test']
lib = getattr(config, 'comet_b200_library', '')
if lib:
    config.available_features.add('b200')
    config.substitutions.append(('%comet_b200_library', lib))
