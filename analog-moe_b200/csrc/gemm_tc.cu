// tcgen05 / TMEM / TMA kernels of the conditional vector-matrix multiply (sm_100a).
//
// cvmm_tc_kernel  (forward and input gradient)
//   Persistent, warp-specialised CTA, one per SM, walking 128-row tiles of the expert-sorted slot
//   list.  Roles:
//     warp 0        lane 0 issues the TMA loads of the prepared bf16 weight tiles (128B swizzle)
//     warp 1        allocates TMEM; lane 0 issues tcgen05.mma (128 x BN x 16, fp32 accumulate in TMEM)
//     warps 2-5     epilogue: tcgen05.ld of the accumulator, one thread per output row, then noise /
//                   ADC / rescale (forward) or clip mask / input-range gradient (backward), stores
//     warps 6-13    operand prologue: gather the tile's rows, clamp / scale / quantise (DAC), convert
//                   to bf16 (hi, and lo when the operand is split) and write the swizzled A tile
//   A and B tiles travel through a ring of shared-memory stages guarded by mbarriers; the
//   accumulator is double-buffered in TMEM so the epilogue of one tile overlaps the MMAs of the next.
//   Split precision issues up to three MMAs per k-step: hi*hi + hi*lo + lo*hi.
//
// dw_tc_kernel (weight gradient)
//   Same structure; the contraction runs over the slots of one expert, both operands are produced
//   by the prologue warps (8x8 register transposes turn row-major rows into K-major tiles), and one
//   CTA owns each (expert, 128 x BN) output tile, so there are no atomics.
//
// Every mbarrier wait is bounded; on a time-out the CTA records AMOE_ERR_WAIT_LIMIT in the status
// word, stops issuing work, drains and frees its TMEM.
#include "gemm_common.cuh"
#include "tc_ptx.cuh"

namespace amoe {
namespace {

using namespace tc;

constexpr int kBM = 128;          // rows per tile (UMMA M)
constexpr int kBK = 64;           // bf16 elements per stage along the contraction (128 bytes)
// dW kernel geometry: 2 control warps, 4 epilogue warps, 8 prologue warps
constexpr int kProdWarps = 8;
constexpr int kEpiWarp0 = 2;
constexpr int kProdWarp0 = 6;
constexpr int kThreads = (kProdWarp0 + kProdWarps) * 32;  // 448
// forward / dX kernel geometry: 2 control warps + 16 worker warps whose split between epilogue and
// prologue is chosen per launch (4, 8 or 12 epilogue warps)
constexpr int kWorkerWarps = 16;
constexpr int kFwdThreads = (2 + kWorkerWarps) * 32;      // 576
constexpr int kMaxEpiGroups = 3;
constexpr int kMaxStages = 8;
constexpr uint32_t kATile = kBM * kBK * 2;  // 16 KiB

// barrier slots
__device__ __forceinline__ uint32_t bar_full_a(uint32_t bars, int s) { return bars + 8u * s; }
__device__ __forceinline__ uint32_t bar_full_b(uint32_t bars, int s) { return bars + 8u * (kMaxStages + s); }
__device__ __forceinline__ uint32_t bar_empty(uint32_t bars, int s) { return bars + 8u * (2 * kMaxStages + s); }
__device__ __forceinline__ uint32_t bar_tfull(uint32_t bars, int b) { return bars + 8u * (3 * kMaxStages + b); }
__device__ __forceinline__ uint32_t bar_tempty(uint32_t bars, int b) { return bars + 8u * (3 * kMaxStages + 2 + b); }
// warp-group rendezvous points (bounded, unlike bar.sync): prologue warps x2, epilogue warps x2
__device__ __forceinline__ uint32_t bar_group(uint32_t bars, int i) { return bars + 8u * (3 * kMaxStages + 4 + i); }
constexpr int kNumBars = 3 * kMaxStages + 8;

struct TileIter {
  const int32_t* off; int E; int e; int64_t before;
  __device__ TileIter(const int32_t* o, int E_) : off(o), E(E_), e(0), before(0) {}
  __device__ bool get(int64_t t, int& ex, int& row0, int& rows) {
    while (e < E) {
      const int beg = off[e], end = off[e + 1];
      const int nt = (end - beg + kBM - 1) / kBM;
      if (t < before + nt) {
        ex = e;
        row0 = beg + static_cast<int>(t - before) * kBM;
        rows = min(kBM, end - row0);
        return true;
      }
      before += nt;
      ++e;
    }
    return false;
  }
};

struct TcParams {
  int E, Kc, Nout;
  int n_epi;   // epilogue warps (multiple of 4); the other worker warps run the operand prologue
  int BN, n_tiles, k_chunks, stages;
  uint32_t tmem_cols, stage_bytes, a_bytes, b_bytes;
  const int32_t* offsets;
  const void* a; int a_dtype; int64_t a_stride; int64_t a_rows; const int32_t* a_row; int a_div;
  const float* ir; const float* a_absmax; float inp_res; int dac; int vec_ok;
  EpiParams epi;
};

// Eight consecutive elements of a row starting at column k (zeros past the row end).
__device__ __forceinline__ void load8(const void* base, int dtype, int64_t row_off, int k, int K, bool vec_ok,
                                      float v[8]) {
  if (k + 8 <= K && vec_ok) {
    if (dtype == AMOE_F32) {
      const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + row_off + k);
      float4 x = __ldg(p), y = __ldg(p + 1);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    } else {
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + row_off + k));
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (k + i < K) ? load_elem(base, dtype, row_off + k + i) : 0.f;
  }
}

template <bool SPLIT>
__device__ __forceinline__ void store8(uint8_t* tile_hi, uint8_t* tile_lo, uint32_t off, const float v[8]) {
  __nv_bfloat16 hi[8], lo[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    hi[i] = __float2bfloat16_rn(v[i]);
    if (SPLIT) lo[i] = __float2bfloat16_rn(v[i] - __bfloat162float(hi[i]));
  }
  *reinterpret_cast<uint4*>(tile_hi + off) =
      make_uint4(pack_bf16x2(hi[0], hi[1]), pack_bf16x2(hi[2], hi[3]), pack_bf16x2(hi[4], hi[5]), pack_bf16x2(hi[6], hi[7]));
  if (SPLIT)
    *reinterpret_cast<uint4*>(tile_lo + off) = make_uint4(pack_bf16x2(lo[0], lo[1]), pack_bf16x2(lo[2], lo[3]),
                                                          pack_bf16x2(lo[4], lo[5]), pack_bf16x2(lo[6], lo[7]));
}

struct SmemView {
  uint8_t* base;       // 1024-aligned
  uint32_t base_u32;
  uint32_t bars;       // shared address of the barrier array
  uint32_t* tmem_ptr;
  volatile int* abort_flag;
};

__device__ __forceinline__ SmemView carve_smem(uint8_t* raw, uint32_t ring_bytes) {
  SmemView s;
  uintptr_t p = reinterpret_cast<uintptr_t>(raw);
  p = (p + 1023) & ~static_cast<uintptr_t>(1023);
  s.base = reinterpret_cast<uint8_t*>(p);
  s.base_u32 = smem_u32(s.base);
  uint8_t* tail = s.base + ring_bytes;
  s.bars = smem_u32(tail);
  s.tmem_ptr = reinterpret_cast<uint32_t*>(tail + 8 * kNumBars);
  s.abort_flag = reinterpret_cast<volatile int*>(tail + 8 * kNumBars + 8);
  return s;
}

__device__ __forceinline__ void setup_cta(const SmemView& s, int stages, uint32_t tmem_cols, int full_a_count,
                                          int tempty_count = 4, int prod_warps = 1, int epi_warps = 1) {
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(bar_full_a(s.bars, i), full_a_count);
      mbar_init(bar_full_b(s.bars, i), 1);
      mbar_init(bar_empty(s.bars, i), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull(s.bars, b), 1);
      mbar_init(bar_tempty(s.bars, b), tempty_count);
    }
    mbar_init(bar_group(s.bars, 0), prod_warps);
    mbar_init(bar_group(s.bars, 1), prod_warps);
    mbar_init(bar_group(s.bars, 2), epi_warps);
    mbar_init(bar_group(s.bars, 3), epi_warps);
    *s.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s.tmem_ptr), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

__device__ __forceinline__ void teardown_cta(const SmemView& s, uint32_t tmem_base, uint32_t tmem_cols) {
  // After a time-out, give copies that may still be in flight time to land before the CTA's
  // shared memory is released.
  if (*s.abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ============================================================================ forward / dX
// Rendezvous of a group of warps on an mbarrier whose arrival count is the number of warps.
// `round` counts the uses of this barrier by the calling warp.  Returns false if the wait gave up.
__device__ __forceinline__ bool group_sync(uint32_t bar, uint32_t round, volatile int* abort_flag, int32_t* status,
                                           int where) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
  bool ok = mbar_wait(bar, round & 1u, abort_flag, status, where);
  return __all_sync(0xffffffffu, ok);
}

// Per-row operand-prologue parameters, staged in shared memory once per tile.
struct __align__(16) RowMeta {
  long long src_off;   // element offset of the source row, or -1 if the row is not to be read
  float ir, am, fast;
  float pad;
};

template <bool A_SPLIT, bool B_SPLIT>
__global__ void __launch_bounds__(kFwdThreads, 1)
cvmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo, TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ RowMeta s_meta[kBM];
  __shared__ float s_dir[kMaxEpiGroups][kBM];
  __shared__ unsigned s_keep[kMaxEpiGroups][kBM];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_prod = kWorkerWarps - p.n_epi;
  setup_cta(sm, p.stages, p.tmem_cols, n_prod, p.n_epi, n_prod, p.n_epi);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.epi.status;

  if (warp == 0) {
    // ---------------------------------------------------------------- weight tiles by TMA
    if (lane == 0) {
      tma_prefetch_desc(&tmap_hi);
      if (B_SPLIT) tma_prefetch_desc(&tmap_lo);
      TileIter ti(p.offsets, p.E);
      uint32_t it = 0;
      bool alive = true;
      for (int64_t t = blockIdx.x; alive; t += gridDim.x) {
        int e, row0, rows;
        if (!ti.get(t, e, row0, rows)) break;
        for (int nt = 0; nt < p.n_tiles && alive; ++nt) {
          for (int kc = 0; kc < p.k_chunks; ++kc, ++it) {
            const int s = it % p.stages;
            const uint32_t ph = (it / p.stages) & 1u;
            if (!mbar_wait(bar_empty(sm.bars, s), ph ^ 1u, sm.abort_flag, status, 1)) { alive = false; break; }
            const uint32_t dst = sm.base_u32 + s * p.stage_bytes + p.a_bytes;
            mbar_arrive_expect_tx(bar_full_b(sm.bars, s), p.b_bytes * (B_SPLIT ? 2u : 1u));
            tma_load_3d(dst, &tmap_hi, bar_full_b(sm.bars, s), kc * kBK, nt * p.BN, e);
            if (B_SPLIT) tma_load_3d(dst + p.b_bytes, &tmap_lo, bar_full_b(sm.bars, s), kc * kBK, nt * p.BN, e);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBM, p.BN);
      TileIter ti(p.offsets, p.E);
      uint32_t it = 0, acc_it = 0;
      bool alive = true;
      for (int64_t t = blockIdx.x; alive; t += gridDim.x) {
        int e, row0, rows;
        if (!ti.get(t, e, row0, rows)) break;
        for (int nt = 0; nt < p.n_tiles && alive; ++nt, ++acc_it) {
          const int buf = acc_it & 1u;
          const uint32_t aph = (acc_it >> 1) & 1u;
          if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 2)) { alive = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
          for (int kc = 0; kc < p.k_chunks; ++kc, ++it) {
            const int s = it % p.stages;
            const uint32_t ph = (it / p.stages) & 1u;
            if (!mbar_wait(bar_full_a(sm.bars, s), ph, sm.abort_flag, status, 3) ||
                !mbar_wait(bar_full_b(sm.bars, s), ph, sm.abort_flag, status, 4)) { alive = false; break; }
            tc_fence_after();
            const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
            const uint64_t da_hi = make_smem_desc_sw128(sa);
            const uint64_t da_lo = make_smem_desc_sw128(sa + kATile);
            const uint64_t db_hi = make_smem_desc_sw128(sa + p.a_bytes);
            const uint64_t db_lo = make_smem_desc_sw128(sa + p.a_bytes + p.b_bytes);
#pragma unroll
            for (int k16 = 0; k16 < kBK / 16; ++k16) {
              const uint64_t adv = static_cast<uint64_t>(k16 * 2);  // 32 bytes >> 4
              umma_bf16(d_tmem, da_hi + adv, db_hi + adv, idesc, (kc | k16) != 0 ? 1u : 0u);
              if (B_SPLIT) umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
              if (A_SPLIT) umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
            }
            umma_commit(bar_empty(sm.bars, s));
          }
          if (alive) umma_commit(bar_tfull(sm.bars, buf));
        }
      }
    }
  } else if (warp < 2 + p.n_epi) {
    // ---------------------------------------------------------------- epilogue
    // TMEM lane quadrant = warp % 4; the warps of one quadrant ("groups") interleave the 16-column chunks.
    const int ew = warp - 2;
    const int q = warp & 3;
    const int grp = ew >> 2;
    const int groups = p.n_epi >> 2;
    const int epi_threads = p.n_epi * 32;
    const int r = q * 32 + lane;
    const int chunks = p.BN / 16;
    TileIter ti(p.offsets, p.E);
    uint32_t acc_it = 0, sync_round = 0;
    bool alive = true;
    (void)epi_threads;
    for (int64_t t = blockIdx.x; alive; t += gridDim.x) {
      int e, row0, rows;
      if (!ti.get(t, e, row0, rows)) break;
      const int64_t i = static_cast<int64_t>(row0) + r;
      RowCtx ctx = epi_row_begin(p.epi, i, e, r < rows);
      for (int nt = 0; nt < p.n_tiles && alive; ++nt, ++acc_it) {
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 5);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * p.BN);
        for (int ch = grp; ch < chunks; ch += groups) {
          float v[16];
          tmem_ld16(taddr + ch * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) epi_quad(p.epi, ctx, nt * p.BN + ch * 16 + 4 * qd, &v[4 * qd]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      }
      if (!alive) break;
      if (p.epi.is_dx && (p.epi.ir_grad || p.epi.keep_count)) {
        // fixed-order combination of the groups' partial row sums
        if (groups > 1) {
          s_dir[grp][r] = ctx.dir_acc;
          s_keep[grp][r] = ctx.valid ? ctx.keep : 0u;
          if (!group_sync(bar_group(sm.bars, 2), sync_round, sm.abort_flag, status, 7)) { alive = false; break; }
          if (grp == 0) {
            float d = s_dir[0][r];
            unsigned kc = s_keep[0][r];
            for (int g = 1; g < groups; ++g) { d += s_dir[g][r]; kc += s_keep[g][r]; }
            ctx.dir_acc = d;
            ctx.keep = kc;
          }
          if (!group_sync(bar_group(sm.bars, 3), sync_round, sm.abort_flag, status, 8)) { alive = false; break; }
          ++sync_round;
        }
        if (grp == 0) {
          epi_row_end(p.epi, ctx, i);
          if (p.epi.keep_count) {
            unsigned kc = ctx.valid ? ctx.keep : 0u;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) kc += __shfl_xor_sync(0xffffffffu, kc, o);
            if (lane == 0 && kc) atomicAdd(p.epi.keep_count, static_cast<unsigned long long>(kc));
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- operand prologue (A tiles)
    const int np = n_prod * 32;
    const int pt = threadIdx.x - (2 + p.n_epi) * 32;  // 0..np-1
    const bool has_ir = p.dac && p.ir != nullptr, has_am = p.dac && p.a_absmax != nullptr;
    const bool quant = p.dac && p.inp_res > 0.f;
    TileIter ti(p.offsets, p.E);
    uint32_t it = 0, sync_round = 0;
    bool alive = true;
    for (int64_t t = blockIdx.x; alive; t += gridDim.x) {
      int e, row0, rows;
      if (!ti.get(t, e, row0, rows)) break;
      // everyone is done with the previous tile's metadata
      if (!group_sync(bar_group(sm.bars, 0), sync_round, sm.abort_flag, status, 9)) break;
      for (int r = pt; r < kBM; r += np) {
        RowMeta m;
        m.src_off = -1; m.ir = 1.f; m.am = 1.f; m.fast = 1.f; m.pad = 0.f;
        if (r < rows) {
          const int64_t i = static_cast<int64_t>(row0) + r;
          const int64_t src = p.a_row[i] / p.a_div;
          if (src < 0 || src >= p.a_rows) {
            report(status, AMOE_ERR_INDEX_RANGE, 20, static_cast<int>(i), static_cast<int>(src));
          } else {
            m.src_off = src * p.a_stride;
            if (has_ir) m.ir = p.ir[i];
            if (has_am) m.am = p.a_absmax[src];
            if (quant) m.fast = dac_fast_mul(has_ir, m.ir, has_am, m.am, p.inp_res);
          }
        }
        s_meta[r] = m;
      }
      if (!group_sync(bar_group(sm.bars, 1), sync_round, sm.abort_flag, status, 10)) break;
      ++sync_round;
      for (int nt = 0; nt < p.n_tiles && alive; ++nt) {
        for (int kc = 0; kc < p.k_chunks; ++kc, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          bool ok = mbar_wait(bar_empty(sm.bars, s), ph ^ 1u, sm.abort_flag, status, 6);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { alive = false; break; }
          uint8_t* a_hi = sm.base + s * p.stage_bytes;
          uint8_t* a_lo = a_hi + kATile;
          // 1024 tasks (128 rows x 8 sixteen-byte chunks), four per thread and round
          for (int base = pt; base < kBM * 8; base += np * 4) {
            float v[4][8];
            RowMeta m[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int task = base + b * np;
              const int r = task >> 3, c = task & 7;
              if (task < kBM * 8) m[b] = s_meta[r]; else m[b].src_off = -1;
              const int k = kc * kBK + c * 8;
              if (m[b].src_off >= 0 && k < p.Kc) {
                load8(p.a, p.a_dtype, m[b].src_off, k, p.Kc, p.vec_ok != 0, v[b]);
              } else {
#pragma unroll
                for (int x = 0; x < 8; ++x) v[b][x] = 0.f;
              }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int task = base + b * np;
              if (task < kBM * 8) {
                const int r = task >> 3, c = task & 7;
                if (p.dac && m[b].src_off >= 0) {
#pragma unroll
                  for (int x = 0; x < 8; ++x) {
                    if (quant)
                      v[b][x] = dac_code(v[b][x], has_ir, m[b].ir, has_am, m[b].am, p.inp_res, m[b].fast);
                    else
                      v[b][x] = dac_normalise(v[b][x], has_ir, m[b].ir, has_am, m[b].am);
                  }
                }
                store8<A_SPLIT>(a_hi, a_lo, sw128_offset(r, c), v[b]);
              }
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full_a(sm.bars, s));
        }
      }
    }
  }
  teardown_cta(sm, tmem_base, p.tmem_cols);
}

// ============================================================================ dW
struct DwParams {
  int E, K, N;
  int BN, m_tiles, n_tiles, stages;
  uint32_t tmem_cols, stage_bytes, b_bytes;
  const int32_t* offsets;
  const void* x; int x_dtype; int64_t x_stride; int64_t x_rows; const int32_t* x_row; const float* ir;
  const void* g; int g_dtype; int64_t g_stride; int64_t g_rows; const int32_t* g_row; int g_div;
  const float* g_scale;
  int x_vec_ok, g_vec_ok;
  float* dw;
  int32_t* status;
};

// Loads an 8(slot) x 8(column) block, transposes it in registers and writes eight 16-byte chunks
// (one per column, eight consecutive slots each) into a K-major swizzled tile.
template <bool SPLIT>
__device__ __forceinline__ void produce_block(const float v[8][8], uint8_t* tile_hi, uint8_t* tile_lo, int row_base,
                                              int sg) {
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    float col[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) col[j] = v[j][m];
    store8<SPLIT>(tile_hi, tile_lo, sw128_offset(row_base + m, sg), col);
  }
}

template <bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1) dw_tc_kernel(DwParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // full_a is the only "data ready" barrier here (both operands come from the prologue warps)
  setup_cta(sm, p.stages, p.tmem_cols, kProdWarps);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.status;
  const int64_t items = static_cast<int64_t>(p.E) * p.m_tiles * p.n_tiles;
  const uint32_t a_total = SPLIT ? 2 * kATile : kATile;

  if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBM, p.BN);
      uint32_t it = 0, acc_it = 0;
      bool alive = true;
      for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
        const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
        const int chunks = (p.offsets[e + 1] - p.offsets[e] + kBK - 1) / kBK;
        if (chunks == 0) continue;
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 12)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
        for (int kc = 0; kc < chunks; ++kc, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          if (!mbar_wait(bar_full_a(sm.bars, s), ph, sm.abort_flag, status, 13)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
          const uint64_t da_hi = make_smem_desc_sw128(sa);
          const uint64_t da_lo = make_smem_desc_sw128(sa + kATile);
          const uint64_t db_hi = make_smem_desc_sw128(sa + a_total);
          const uint64_t db_lo = make_smem_desc_sw128(sa + a_total + p.b_bytes);
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            const uint64_t adv = static_cast<uint64_t>(k16 * 2);
            umma_bf16(d_tmem, da_hi + adv, db_hi + adv, idesc, (kc | k16) != 0 ? 1u : 0u);
            if (SPLIT) {
              umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
              umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
            }
          }
          umma_commit(bar_empty(sm.bars, s));
        }
        if (alive) umma_commit(bar_tfull(sm.bars, buf));
        ++acc_it;
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kProdWarp0) {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    uint32_t acc_it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
      const int nt = static_cast<int>(w % p.n_tiles);
      const int mt = static_cast<int>((w / p.n_tiles) % p.m_tiles);
      const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
      const int chunks = (p.offsets[e + 1] - p.offsets[e] + kBK - 1) / kBK;
      const int m = mt * kBM + r;
      const int n0 = nt * p.BN;
      float* dst = p.dw + (static_cast<int64_t>(e) * p.K + m) * p.N;
      if (chunks == 0) {
        if (m < p.K)
          for (int n = n0; n < min(n0 + p.BN, p.N); ++n) dst[n] = 0.f;
        continue;
      }
      const int buf = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 15);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * p.BN);
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + c0, v);
        tmem_ld_wait();
        if (m < p.K) {
          const int n = n0 + c0;
          if (n + 16 <= p.N && ((reinterpret_cast<uintptr_t>(dst + n) & 15u) == 0)) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
              *reinterpret_cast<float4*>(dst + n + 4 * x) = make_float4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
          } else {
#pragma unroll
            for (int x = 0; x < 16; ++x)
              if (n + x < p.N) dst[n + x] = v[x];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      ++acc_it;
    }
  } else if (warp >= kProdWarp0) {
    const int pt = threadIdx.x - kProdWarp0 * 32;  // 0..255
    const bool is_b = pt >= 128;
    const int u = pt & 127;
    const int sg = u & 7;    // slot group: slots sg*8 .. sg*8+7 of the stage
    const int cg = u >> 3;   // column group: columns cg*8 .. cg*8+7 of the tile
    uint32_t it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
      const int nt = static_cast<int>(w % p.n_tiles);
      const int mt = static_cast<int>((w / p.n_tiles) % p.m_tiles);
      const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
      const int beg = p.offsets[e], end = p.offsets[e + 1];
      const int chunks = (end - beg + kBK - 1) / kBK;
      const int col0 = is_b ? nt * p.BN + cg * 8 : mt * kBM + cg * 8;
      const int col_lim = is_b ? p.N : p.K;
      const bool active = is_b ? (cg * 8 < p.BN) : true;
      for (int kc = 0; kc < chunks; ++kc, ++it) {
        const int s = it % p.stages;
        const uint32_t ph = (it / p.stages) & 1u;
        bool ok = mbar_wait(bar_empty(sm.bars, s), ph ^ 1u, sm.abort_flag, status, 16);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        uint8_t* stage = sm.base + s * p.stage_bytes;
        if (active) {
          float v[8][8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = beg + kc * kBK + sg * 8 + j;
            bool okr = i < end && col0 < col_lim;
            if (okr) {
              if (!is_b) {
                const int64_t xr = p.x_row[i];
                if (xr < 0 || xr >= p.x_rows) {
                  report(status, AMOE_ERR_INDEX_RANGE, 30, i, static_cast<int>(xr));
                  okr = false;
                } else {
                  load8(p.x, p.x_dtype, xr * p.x_stride, col0, p.K, p.x_vec_ok != 0, v[j]);
                  if (p.ir) {
                    const float r = p.ir[i];
#pragma unroll
                    for (int x = 0; x < 8; ++x) v[j][x] = clamp_ir(v[j][x], r);
                  }
                }
              } else {
                const int64_t gr = p.g_row[i];
                if (gr < 0 || gr / p.g_div >= p.g_rows) {
                  report(status, AMOE_ERR_INDEX_RANGE, 31, i, static_cast<int>(gr));
                  okr = false;
                } else {
                  load8(p.g, p.g_dtype, (gr / p.g_div) * p.g_stride, col0, p.N, p.g_vec_ok != 0, v[j]);
                  if (p.g_scale) {
                    const float sc = p.g_scale[gr];
#pragma unroll
                    for (int x = 0; x < 8; ++x) v[j][x] *= sc;
                  }
                }
              }
            }
            if (!okr) {
#pragma unroll
              for (int x = 0; x < 8; ++x) v[j][x] = 0.f;
            }
          }
          if (!is_b)
            produce_block<SPLIT>(v, stage, stage + kATile, cg * 8, sg);
          else
            produce_block<SPLIT>(v, stage + a_total, stage + a_total + p.b_bytes, cg * 8, sg);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full_a(sm.bars, s));
      }
    }
  }
  teardown_cta(sm, tmem_base, p.tmem_cols);
}

// ---------------------------------------------------------------------------- dW, MN-major operands
// The contraction index of dW is the slot, which is the slow index of both row-major inputs.  The
// tensor core takes such operands directly ("MN-major"): a stage holds 64 slots as 64 rows of 128 bytes
// per block of 64 columns, so the prologue converts and stores 16-byte chunks without transposing.
struct DwMnParams {
  int E, K, N;
  int BN, m_tiles, n_tiles, stages;
  uint32_t tmem_cols, stage_bytes, a_bytes, b_bytes;   // a_bytes/b_bytes: one precision term of A / B
  const int32_t* offsets;
  const void* x; int x_dtype; int64_t x_stride; int64_t x_rows; const int32_t* x_row; const float* ir;
  const void* g; int g_dtype; int64_t g_stride; int64_t g_rows; const int32_t* g_row; int g_div;
  const float* g_scale;
  int x_vec_ok, g_vec_ok;
  float* dw;
  int32_t* status;
};

constexpr int kDwProdWarps = 12;
constexpr uint32_t kMnBlock = kBK * 128;   // 64 rows x 128 bytes

template <bool SPLIT>
__global__ void __launch_bounds__(kFwdThreads, 1) dw_tc_mn_kernel(DwMnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup_cta(sm, p.stages, p.tmem_cols, kDwProdWarps, 4);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.status;
  const int64_t items = static_cast<int64_t>(p.E) * p.m_tiles * p.n_tiles;
  const uint32_t a_total = SPLIT ? 2 * p.a_bytes : p.a_bytes;

  if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16_mn(kBM, p.BN);
      uint32_t it = 0, acc_it = 0;
      bool alive = true;
      for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
        const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
        const int chunks = (p.offsets[e + 1] - p.offsets[e] + kBK - 1) / kBK;
        if (chunks == 0) continue;
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 12)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
        for (int kc = 0; kc < chunks; ++kc, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          if (!mbar_wait(bar_full_a(sm.bars, s), ph, sm.abort_flag, status, 13)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
          const uint64_t da_hi = make_smem_desc_mn_sw128(sa, kMnBlock);
          const uint64_t da_lo = make_smem_desc_mn_sw128(sa + p.a_bytes, kMnBlock);
          const uint64_t db_hi = make_smem_desc_mn_sw128(sa + a_total, kMnBlock);
          const uint64_t db_lo = make_smem_desc_mn_sw128(sa + a_total + p.b_bytes, kMnBlock);
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            const uint64_t adv = static_cast<uint64_t>(k16 * (16 * 128 / 16));  // 16 rows of 128 bytes, >> 4
            umma_bf16(d_tmem, da_hi + adv, db_hi + adv, idesc, (kc | k16) != 0 ? 1u : 0u);
            if (SPLIT) {
              umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
              umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
            }
          }
          umma_commit(bar_empty(sm.bars, s));
        }
        if (alive) umma_commit(bar_tfull(sm.bars, buf));
        ++acc_it;
      }
    }
  } else if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    uint32_t acc_it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
      const int nt = static_cast<int>(w % p.n_tiles);
      const int mt = static_cast<int>((w / p.n_tiles) % p.m_tiles);
      const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
      const int chunks = (p.offsets[e + 1] - p.offsets[e] + kBK - 1) / kBK;
      const int m = mt * kBM + r;
      const int n0 = nt * p.BN;
      float* dst = p.dw + (static_cast<int64_t>(e) * p.K + m) * p.N;
      if (chunks == 0) {
        if (m < p.K)
          for (int n = n0; n < min(n0 + p.BN, p.N); ++n) dst[n] = 0.f;
        continue;
      }
      const int buf = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 15);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * p.BN);
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + c0, v);
        tmem_ld_wait();
        if (m < p.K) {
          const int n = n0 + c0;
          if (n + 16 <= p.N && ((reinterpret_cast<uintptr_t>(dst + n) & 15u) == 0)) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
              *reinterpret_cast<float4*>(dst + n + 4 * x) = make_float4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
          } else {
#pragma unroll
            for (int x = 0; x < 16; ++x)
              if (n + x < p.N) dst[n + x] = v[x];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      ++acc_it;
    }
  } else if (warp >= 6) {
    constexpr int np = kDwProdWarps * 32;               // 384
    const int pt = threadIdx.x - 6 * 32;
    const int a_chunks = kBM / 8;                        // 16 sixteen-byte chunks per slot row of A
    const int b_chunks = (p.BN + 7) / 8;
    const int a_tasks = kBK * a_chunks;                  // 1024
    const int tasks = a_tasks + kBK * b_chunks;
    uint32_t it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; w < items && alive; w += gridDim.x) {
      const int nt = static_cast<int>(w % p.n_tiles);
      const int mt = static_cast<int>((w / p.n_tiles) % p.m_tiles);
      const int e = static_cast<int>(w / (p.m_tiles * p.n_tiles));
      const int beg = p.offsets[e], end = p.offsets[e + 1];
      const int chunks = (end - beg + kBK - 1) / kBK;
      for (int kc = 0; kc < chunks; ++kc, ++it) {
        const int s = it % p.stages;
        const uint32_t ph = (it / p.stages) & 1u;
        bool ok = mbar_wait(bar_empty(sm.bars, s), ph ^ 1u, sm.abort_flag, status, 16);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        uint8_t* stage = sm.base + s * p.stage_bytes;
        const int i0 = beg + kc * kBK;
        for (int base = pt; base < tasks; base += np * 3) {
          float v[3][8];
          int where[3];       // byte offset inside the operand term, or -1
          bool isb[3];
#pragma unroll
          for (int b = 0; b < 3; ++b) {
            const int task = base + b * np;
            where[b] = -1;
            isb[b] = task >= a_tasks;
#pragma unroll
            for (int x = 0; x < 8; ++x) v[b][x] = 0.f;
            if (task < tasks) {
              const int tt = isb[b] ? task - a_tasks : task;
              const int cpr = isb[b] ? b_chunks : a_chunks;
              const int r = tt / cpr, c = tt - r * cpr;
              where[b] = (c >> 3) * static_cast<int>(kMnBlock) + static_cast<int>(sw128_offset(r, c & 7));
              const int i = i0 + r;
              if (i < end) {
                if (!isb[b]) {
                  const int col = mt * kBM + c * 8;
                  const int64_t xr = p.x_row[i];
                  if (xr < 0 || xr >= p.x_rows) {
                    report(status, AMOE_ERR_INDEX_RANGE, 30, i, static_cast<int>(xr));
                  } else if (col < p.K) {
                    load8(p.x, p.x_dtype, xr * p.x_stride, col, p.K, p.x_vec_ok != 0, v[b]);
                    if (p.ir) {
                      const float rr = p.ir[i];
#pragma unroll
                      for (int x = 0; x < 8; ++x) v[b][x] = clamp_ir(v[b][x], rr);
                    }
                  }
                } else {
                  const int col = nt * p.BN + c * 8;
                  const int64_t gr = p.g_row[i];
                  if (gr < 0 || gr / p.g_div >= p.g_rows) {
                    report(status, AMOE_ERR_INDEX_RANGE, 31, i, static_cast<int>(gr));
                  } else if (col < p.N) {
                    load8(p.g, p.g_dtype, (gr / p.g_div) * p.g_stride, col, p.N, p.g_vec_ok != 0, v[b]);
                    if (p.g_scale) {
                      const float sc = p.g_scale[gr];
#pragma unroll
                      for (int x = 0; x < 8; ++x) v[b][x] *= sc;
                    }
                  }
                }
              }
            }
          }
#pragma unroll
          for (int b = 0; b < 3; ++b) {
            if (where[b] >= 0) {
              uint8_t* hi = stage + (isb[b] ? a_total : 0u);
              uint8_t* lo = hi + (isb[b] ? p.b_bytes : p.a_bytes);
              store8<SPLIT>(hi, lo, static_cast<uint32_t>(where[b]), v[b]);
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full_a(sm.bars, s));
      }
    }
  }
  teardown_cta(sm, tmem_base, p.tmem_cols);
}

uint32_t pow2_cols(int need) {
  uint32_t c = 32;
  while (static_cast<int>(c) < need) c <<= 1;
  return c;
}

constexpr uint32_t kSmemBudget = 192 * 1024;  // ring budget; barriers and alignment slack come on top
constexpr uint32_t kSmemExtra = 1024 + 8 * kNumBars + 64;

}  // namespace

// ---------------------------------------------------------------------------- host: tensor maps
int encode_tmap_bf16_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box0,
                        uint32_t box1) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    AMOE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    if (sym == nullptr || qres != cudaDriverEntryPointSuccess) {
      set_last_error("cuTensorMapEncodeTiled entry point not found", cudaErrorUnknown);
      return AMOE_ERR_CUDA;
    }
    fn = reinterpret_cast<EncodeFn>(sym);
  }
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed", cudaErrorInvalidValue);
    return AMOE_ERR_CUDA;
  }
  return AMOE_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_cvmm_tc(const amoe_cvmm_args* a, bool is_dx, const EpiParams& epi_in, cudaStream_t stream) {
  int s = amoe_check_device();
  if (s != AMOE_OK) return s;
  TcParams p{};
  p.E = a->E;
  p.Kc = is_dx ? a->N : a->K;
  p.Nout = is_dx ? a->K : a->N;
  const int n_pad = round_up(p.Nout, 16);
  const int k_pad = round_up(p.Kc, 64);
  p.n_tiles = (n_pad + 255) / 256;
  p.BN = round_up((n_pad + p.n_tiles - 1) / p.n_tiles, 16);
  p.k_chunks = k_pad / kBK;
  p.offsets = a->expert_offsets;
  p.a = a->a; p.a_dtype = a->a_dtype; p.a_stride = a->a_stride; p.a_rows = a->a_rows; p.a_row = a->a_row;
  p.a_div = a->a_row_div < 1 ? 1 : a->a_row_div;
  p.dac = is_dx ? 0 : 1;
  p.ir = is_dx ? nullptr : a->ir;
  p.a_absmax = is_dx ? nullptr : a->a_absmax;
  p.inp_res = is_dx ? -1.f : a->inp_res;
  const int esz = a->a_dtype == AMOE_F32 ? 4 : 2;
  p.vec_ok = aligned16(a->a) && ((a->a_stride * esz) % 16 == 0);
  p.epi = epi_in;
  const bool quant = p.dac && p.inp_res > 0.f;
  // Integer DAC codes up to 256 in magnitude are exact in bf16; anything else needs the hi+lo pair
  // when split precision is asked for.  bf16 inputs that are not quantised are exact as they are.
  bool a_split = a->precision == AMOE_PREC_SPLIT;
  if (quant && p.inp_res >= 1.0f / 256.0f) a_split = false;
  if (!p.dac && a->a_dtype == AMOE_BF16) a_split = false;
  const bool b_split = a->precision == AMOE_PREC_SPLIT && a->w_lo != nullptr;
  p.epi.acc_mul = quant ? p.inp_res : 1.f;

  p.a_bytes = a_split ? 2 * kATile : kATile;
  p.b_bytes = static_cast<uint32_t>(p.BN) * 128u;
  p.stage_bytes = p.a_bytes + p.b_bytes * (b_split ? 2u : 1u);
  p.stage_bytes = (p.stage_bytes + 1023u) & ~1023u;
  p.stages = static_cast<int>(kSmemBudget / p.stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  AMOE_REQUIRE(p.stages >= 2, AMOE_ERR_UNSUPPORTED);
  p.tmem_cols = pow2_cols(2 * p.BN);
  {
    // Split the 16 worker warps between epilogue and prologue by estimated instruction counts.
    const double per_prod = (quant ? 13.0 : (p.dac ? 30.0 : 4.0)) + (a_split ? 6.0 : 2.0);
    double per_epi = 10.0;
    if (!is_dx) per_epi += (a->noise_std > 0.f ? 26.0 : 0.0) + (a->noise ? 2.0 : 0.0) + (p.epi.adc.on ? 9.0 : 0.0) +
                           (a->out_codes ? 3.0 : 0.0);
    else per_epi += a->x_ref ? 12.0 : 0.0;
    const double work_p = static_cast<double>(p.n_tiles) * p.k_chunks * kBK * per_prod;
    const double work_e = static_cast<double>(p.n_tiles) * p.BN * per_epi;
    double best = 1e300;
    for (int ne = 4; ne <= 12; ne += 4) {
      const double t = fmax(work_p / (kWorkerWarps - ne), work_e / ne);
      if (t < best) { best = t; p.n_epi = ne; }
    }
  }

  CUtensorMap m_hi, m_lo;
  s = encode_tmap_bf16_3d(&m_hi, a->w_hi, static_cast<uint64_t>(k_pad), static_cast<uint64_t>(n_pad),
                          static_cast<uint64_t>(a->E), kBK, static_cast<uint32_t>(p.BN));
  if (s != AMOE_OK) return s;
  m_lo = m_hi;
  if (b_split) {
    s = encode_tmap_bf16_3d(&m_lo, a->w_lo, static_cast<uint64_t>(k_pad), static_cast<uint64_t>(n_pad),
                            static_cast<uint64_t>(a->E), kBK, static_cast<uint32_t>(p.BN));
    if (s != AMOE_OK) return s;
  }
  const uint32_t smem = p.stages * p.stage_bytes + kSmemExtra;
  const int64_t max_tiles = (a->P + kBM - 1) / kBM + a->E;
  const int grid = static_cast<int>(max_tiles < sm_count() ? max_tiles : sm_count());
#define AMOE_LAUNCH_TC(AS, BS)                                                                                  \
  do {                                                                                                          \
    AMOE_CUDA(cudaFuncSetAttribute(cvmm_tc_kernel<AS, BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    cvmm_tc_kernel<AS, BS><<<grid, kFwdThreads, smem, stream>>>(m_hi, m_lo, p);                                 \
  } while (0)
  if (a_split && b_split) AMOE_LAUNCH_TC(true, true);
  else if (a_split) AMOE_LAUNCH_TC(true, false);
  else if (b_split) AMOE_LAUNCH_TC(false, true);
  else AMOE_LAUNCH_TC(false, false);
#undef AMOE_LAUNCH_TC
  AMOE_LAUNCH_CHECK("cvmm_tc");
  return AMOE_OK;
}

int launch_dw_tc(const amoe_dw_args* a, cudaStream_t stream) {
  int s = amoe_check_device();
  if (s != AMOE_OK) return s;
  DwMnParams p{};
  p.E = a->E; p.K = a->K; p.N = a->N;
  const int n_pad = round_up(a->N, 16);
  p.n_tiles = (n_pad + 127) / 128;
  p.BN = round_up((n_pad + p.n_tiles - 1) / p.n_tiles, 16);
  p.m_tiles = (a->K + kBM - 1) / kBM;
  p.offsets = a->expert_offsets;
  p.x = a->x; p.x_dtype = a->x_dtype; p.x_stride = a->x_stride; p.x_rows = a->x_rows; p.x_row = a->x_row;
  p.ir = a->ir;
  p.g = a->g; p.g_dtype = a->g_dtype; p.g_stride = a->g_stride; p.g_rows = a->g_rows; p.g_row = a->g_row;
  p.g_div = a->g_div < 1 ? 1 : a->g_div; p.g_scale = a->g_scale;
  p.x_vec_ok = aligned16(a->x) && ((a->x_stride * (a->x_dtype == AMOE_F32 ? 4 : 2)) % 16 == 0);
  p.g_vec_ok = aligned16(a->g) && ((a->g_stride * (a->g_dtype == AMOE_F32 ? 4 : 2)) % 16 == 0);
  p.dw = a->dw; p.status = a->dev_status;
  // bf16 inputs are exact in one term; fp32 inputs are split unless the caller asked for the fast mode
  const bool split = a->precision == AMOE_PREC_SPLIT && !(a->x_dtype == AMOE_BF16 && a->g_dtype == AMOE_BF16 && !a->g_scale);
  p.a_bytes = 2 * kMnBlock;                                             // 128 columns = 2 blocks
  p.b_bytes = static_cast<uint32_t>((p.BN + 63) / 64) * kMnBlock;
  p.stage_bytes = (split ? 2u : 1u) * (p.a_bytes + p.b_bytes);
  p.stages = static_cast<int>(kSmemBudget / p.stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  AMOE_REQUIRE(p.stages >= 2, AMOE_ERR_UNSUPPORTED);
  p.tmem_cols = pow2_cols(2 * p.BN);
  const uint32_t smem = p.stages * p.stage_bytes + kSmemExtra;
  const int64_t items = static_cast<int64_t>(a->E) * p.m_tiles * p.n_tiles;
  const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
  if (split) {
    AMOE_CUDA(cudaFuncSetAttribute(dw_tc_mn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dw_tc_mn_kernel<true><<<grid, kFwdThreads, smem, stream>>>(p);
  } else {
    AMOE_CUDA(cudaFuncSetAttribute(dw_tc_mn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dw_tc_mn_kernel<false><<<grid, kFwdThreads, smem, stream>>>(p);
  }
  AMOE_LAUNCH_CHECK("dw_tc");
  return AMOE_OK;
}

}  // namespace amoe
