// Pieces shared by the CVMM kernels: tile lookup and host-side launch declarations.
#pragma once
#include "epilogue.cuh"

namespace amoe {

// The sorted slot list is cut into row tiles that never straddle two experts: expert e owns
// ceil(count_e / tile_m) tiles.  Finds tile number `t`; e = -1 if t is past the last tile.
__device__ __forceinline__ void find_tile(const int32_t* __restrict__ offsets, int E, int tile_m, int64_t t, int& e,
                                          int& row0, int& rows) {
  int64_t before = 0;
  for (int x = 0; x < E; ++x) {
    const int beg = offsets[x], end = offsets[x + 1];
    const int nt = (end - beg + tile_m - 1) / tile_m;
    if (t < before + nt) {
      e = x;
      row0 = beg + static_cast<int>(t - before) * tile_m;
      rows = min(tile_m, end - row0);
      return;
    }
    before += nt;
  }
  e = -1; row0 = 0; rows = 0;
}

int launch_cvmm_simt(const amoe_cvmm_args* a, bool is_dx, const EpiParams& epi, cudaStream_t stream);
int launch_dw_simt(const amoe_dw_args* a, cudaStream_t stream);
int launch_cvmm_tc(const amoe_cvmm_args* a, bool is_dx, const EpiParams& epi, cudaStream_t stream);
int launch_dw_tc(const amoe_dw_args* a, cudaStream_t stream);
// `expected` (0 = P): the slot count the segment size is tuned for, when P is only an upper bound.
size_t dw_tc_workspace_bytes(int64_t P, int64_t expected, int E, int K, int N);

}  // namespace amoe
