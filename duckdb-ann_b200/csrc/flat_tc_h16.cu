// The tensor-core flat kernel a third time, over 16-bit operands: rows stored as fp16 or bf16
// (the reduced-precision storage of faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-43), queries
// rounded or split into the same type, tcgen05.mma kind::f16 with fp32 accumulation in tensor memory.
// K blocks of 64 elements are the same 128-byte swizzled rows as in flat_tc_bk32.cu, so the ring, the
// static schedule and the pair mode carry over unchanged.  Only launch_flat_tc_h16 comes out of this
// translation unit.
#define ANN_TC_VARIANT_H16 1
#include "flat_tc.cu"
