// placeholder, replaced below
#include "common.cuh"
extern "C" int conef_tc_supported(void) { return 0; }
