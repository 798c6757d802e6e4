// Instantiations of the direct lookup kernel for 4-bit rows (see
// spmdm_direct.cuh).  One translation unit per bit rate keeps the build
// parallel.
#include "spmdm_direct.cuh"

namespace fbgemm_b200 {

const direct::Variant* direct_variants_4(int* count) {
  using namespace direct;
  static const Variant v[] = {
      {spmdm_direct_kernel<4, 4, 2, 1>, spmdm_direct_multi_kernel<4, 4, 2, 1>, spmdm_direct_compact_kernel<4, 4, 2, 1>,
       spmdm_direct_compact_multi_kernel<4, 4, 2, 1>, 4, 2, 1},
      {spmdm_direct_kernel<4, 4, 4, 1>, spmdm_direct_multi_kernel<4, 4, 4, 1>, spmdm_direct_compact_kernel<4, 4, 4, 1>,
       spmdm_direct_compact_multi_kernel<4, 4, 4, 1>, 4, 4, 1},
      {spmdm_direct_kernel<4, 4, 8, 1>, spmdm_direct_multi_kernel<4, 4, 8, 1>, spmdm_direct_compact_kernel<4, 4, 8, 1>,
       spmdm_direct_compact_multi_kernel<4, 4, 8, 1>, 4, 8, 1},
      {spmdm_direct_kernel<4, 4, 16, 1>, spmdm_direct_multi_kernel<4, 4, 16, 1>, spmdm_direct_compact_kernel<4, 4, 16, 1>,
       spmdm_direct_compact_multi_kernel<4, 4, 16, 1>, 4, 16, 1},
      {spmdm_direct_kernel<4, 4, 32, 1>, spmdm_direct_multi_kernel<4, 4, 32, 1>, spmdm_direct_compact_kernel<4, 4, 32, 1>,
       spmdm_direct_compact_multi_kernel<4, 4, 32, 1>, 4, 32, 1},
      {spmdm_direct_kernel<4, 4, 2, 2>, spmdm_direct_multi_kernel<4, 4, 2, 2>, spmdm_direct_compact_kernel<4, 4, 2, 2>,
       spmdm_direct_compact_multi_kernel<4, 4, 2, 2>, 4, 2, 2},
      {spmdm_direct_kernel<4, 4, 4, 2>, spmdm_direct_multi_kernel<4, 4, 4, 2>, spmdm_direct_compact_kernel<4, 4, 4, 2>,
       spmdm_direct_compact_multi_kernel<4, 4, 4, 2>, 4, 4, 2},
      {spmdm_direct_kernel<4, 4, 8, 2>, spmdm_direct_multi_kernel<4, 4, 8, 2>, spmdm_direct_compact_kernel<4, 4, 8, 2>,
       spmdm_direct_compact_multi_kernel<4, 4, 8, 2>, 4, 8, 2},
      {spmdm_direct_kernel<4, 4, 16, 2>, spmdm_direct_multi_kernel<4, 4, 16, 2>, spmdm_direct_compact_kernel<4, 4, 16, 2>,
       spmdm_direct_compact_multi_kernel<4, 4, 16, 2>, 4, 16, 2},
      {spmdm_direct_kernel<4, 4, 32, 2>, spmdm_direct_multi_kernel<4, 4, 32, 2>, spmdm_direct_compact_kernel<4, 4, 32, 2>,
       spmdm_direct_compact_multi_kernel<4, 4, 32, 2>, 4, 32, 2},
      {spmdm_direct_kernel<4, 4, 2, 4>, spmdm_direct_multi_kernel<4, 4, 2, 4>, spmdm_direct_compact_kernel<4, 4, 2, 4>,
       spmdm_direct_compact_multi_kernel<4, 4, 2, 4>, 4, 2, 4},
      {spmdm_direct_kernel<4, 4, 4, 4>, spmdm_direct_multi_kernel<4, 4, 4, 4>, spmdm_direct_compact_kernel<4, 4, 4, 4>,
       spmdm_direct_compact_multi_kernel<4, 4, 4, 4>, 4, 4, 4},
      {spmdm_direct_kernel<4, 4, 8, 4>, spmdm_direct_multi_kernel<4, 4, 8, 4>, spmdm_direct_compact_kernel<4, 4, 8, 4>,
       spmdm_direct_compact_multi_kernel<4, 4, 8, 4>, 4, 8, 4},
      {spmdm_direct_kernel<4, 4, 16, 4>, spmdm_direct_multi_kernel<4, 4, 16, 4>, spmdm_direct_compact_kernel<4, 4, 16, 4>,
       spmdm_direct_compact_multi_kernel<4, 4, 16, 4>, 4, 16, 4},
      {spmdm_direct_kernel<4, 4, 32, 4>, spmdm_direct_multi_kernel<4, 4, 32, 4>, spmdm_direct_compact_kernel<4, 4, 32, 4>,
       spmdm_direct_compact_multi_kernel<4, 4, 32, 4>, 4, 32, 4},
      {spmdm_direct_kernel<4, 8, 2, 1>, spmdm_direct_multi_kernel<4, 8, 2, 1>, spmdm_direct_compact_kernel<4, 8, 2, 1>,
       spmdm_direct_compact_multi_kernel<4, 8, 2, 1>, 8, 2, 1},
      {spmdm_direct_kernel<4, 8, 4, 1>, spmdm_direct_multi_kernel<4, 8, 4, 1>, spmdm_direct_compact_kernel<4, 8, 4, 1>,
       spmdm_direct_compact_multi_kernel<4, 8, 4, 1>, 8, 4, 1},
      {spmdm_direct_kernel<4, 8, 8, 1>, spmdm_direct_multi_kernel<4, 8, 8, 1>, spmdm_direct_compact_kernel<4, 8, 8, 1>,
       spmdm_direct_compact_multi_kernel<4, 8, 8, 1>, 8, 8, 1},
      {spmdm_direct_kernel<4, 8, 16, 1>, spmdm_direct_multi_kernel<4, 8, 16, 1>, spmdm_direct_compact_kernel<4, 8, 16, 1>,
       spmdm_direct_compact_multi_kernel<4, 8, 16, 1>, 8, 16, 1},
      {spmdm_direct_kernel<4, 8, 32, 1>, spmdm_direct_multi_kernel<4, 8, 32, 1>, spmdm_direct_compact_kernel<4, 8, 32, 1>,
       spmdm_direct_compact_multi_kernel<4, 8, 32, 1>, 8, 32, 1},
      {spmdm_direct_kernel<4, 8, 2, 2>, spmdm_direct_multi_kernel<4, 8, 2, 2>, spmdm_direct_compact_kernel<4, 8, 2, 2>,
       spmdm_direct_compact_multi_kernel<4, 8, 2, 2>, 8, 2, 2},
      {spmdm_direct_kernel<4, 8, 4, 2>, spmdm_direct_multi_kernel<4, 8, 4, 2>, spmdm_direct_compact_kernel<4, 8, 4, 2>,
       spmdm_direct_compact_multi_kernel<4, 8, 4, 2>, 8, 4, 2},
      {spmdm_direct_kernel<4, 8, 8, 2>, spmdm_direct_multi_kernel<4, 8, 8, 2>, spmdm_direct_compact_kernel<4, 8, 8, 2>,
       spmdm_direct_compact_multi_kernel<4, 8, 8, 2>, 8, 8, 2},
      {spmdm_direct_kernel<4, 8, 16, 2>, spmdm_direct_multi_kernel<4, 8, 16, 2>, spmdm_direct_compact_kernel<4, 8, 16, 2>,
       spmdm_direct_compact_multi_kernel<4, 8, 16, 2>, 8, 16, 2},
      {spmdm_direct_kernel<4, 8, 32, 2>, spmdm_direct_multi_kernel<4, 8, 32, 2>, spmdm_direct_compact_kernel<4, 8, 32, 2>,
       spmdm_direct_compact_multi_kernel<4, 8, 32, 2>, 8, 32, 2},
  };
  *count = (int)(sizeof(v) / sizeof(v[0]));
  return v;
}

}  // namespace fbgemm_b200
