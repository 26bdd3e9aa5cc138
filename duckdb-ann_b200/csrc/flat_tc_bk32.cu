// The tensor-core flat kernel once more, with K blocks of 32 floats (one 128-byte swizzled row per
// operand row, two 96 KB stages = four stages of hi planes): the build the screened search uses.
// Only launch_flat_tc_bk32 comes out of this translation unit.
#define ANN_TC_VARIANT_BK32 1
#include "flat_tc.cu"
