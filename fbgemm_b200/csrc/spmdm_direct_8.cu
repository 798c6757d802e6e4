// Instantiations of the direct lookup kernel for 8-bit rows (see
// spmdm_direct.cuh).  One translation unit per bit rate keeps the build
// parallel.  Listed are the (VEC, LPB, CPL) combinations the dispatcher can
// pick (pick_direct in spmdm_kernels.cu), each in its two addressing forms.
#include "spmdm_direct.cuh"

namespace fbgemm_b200 {

#define V(VEC, LPB, CPL)                                                                                            \
  {{spmdm_direct_kernel<8, VEC, LPB, CPL, false>, spmdm_direct_kernel<8, VEC, LPB, CPL, true>},                         \
   {spmdm_direct_multi_kernel<8, VEC, LPB, CPL, false>, spmdm_direct_multi_kernel<8, VEC, LPB, CPL, true>},             \
   {spmdm_direct_compact_kernel<8, VEC, LPB, CPL, false>, spmdm_direct_compact_kernel<8, VEC, LPB, CPL, true>},         \
   {spmdm_direct_compact_multi_kernel<8, VEC, LPB, CPL, false>, spmdm_direct_compact_multi_kernel<8, VEC, LPB, CPL, true>}, \
   VEC, LPB, CPL}

const direct::Variant* direct_variants_8(int* count) {
  using namespace direct;
  static const Variant v[] = {
      V(4, 4, 1), V(4, 4, 2), V(4, 4, 4), V(4, 4, 8), V(4, 8, 8), V(4, 16, 4), V(4, 32, 4), V(4, 32, 8),
      V(8, 4, 1), V(8, 4, 2), V(8, 4, 4), V(8, 8, 4), V(8, 16, 2), V(8, 32, 2), V(8, 32, 4),
#ifdef FBGEMM_B200_TUNING
      V(4, 8, 1), V(4, 8, 2), V(4, 8, 4), V(4, 16, 1), V(4, 16, 2), V(4, 16, 8),
      V(8, 8, 1), V(8, 8, 2), V(8, 16, 1), V(8, 16, 4), V(8, 32, 1),
#endif
  };
  *count = (int)(sizeof(v) / sizeof(v[0]));
  return v;
}

#undef V

}  // namespace fbgemm_b200
