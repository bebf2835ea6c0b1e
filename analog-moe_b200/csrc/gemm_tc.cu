// tcgen05 / TMEM / TMA kernels of the conditional vector-matrix multiply (sm_100a).
//
// cvmm_tc_kernel  (forward and input gradient)
//   Persistent, warp-specialised CTA, one per SM, walking 128-row tiles of the expert-sorted slot
//   list.  24 warps:
//     warp 0        lane 0 issues the TMA loads of the prepared bf16 weight tiles (128B swizzle)
//     warp 1        allocates TMEM; lane 0 issues tcgen05.mma (128 x BN x 16, fp32 accumulate in TMEM)
//     22 workers    split per launch between
//       epilogue:   tcgen05.ld of the accumulator, one thread per output row and share of the
//                   columns, then noise / ADC / rescale (forward) or clip mask / input-range
//                   gradient (backward), stores
//       prologue:   gather the tile's rows, clamp / scale / quantise (DAC), convert to bf16 (hi, and
//                   lo when the operand is split) and write the swizzled K-major A tile; two groups of
//                   prologue warps take alternate ring stages; optionally the clamped rows are also
//                   written out as the bf16 operand cache of the later weight gradient
//   When the A operand already exists as such a cache (the up-projection's dX reads the hidden
//   gradient the down-projection's dX left behind) warp 0 loads it by TMA and there is no prologue.
//   A and B tiles travel through a ring of shared-memory stages guarded by mbarriers; the
//   accumulator is double-buffered in TMEM so the epilogue of one tile overlaps the MMAs of the next.
//   Split precision issues up to three MMAs per k-step: hi*hi + hi*lo + lo*hi.
//   The kernel is instantiated per DAC mode, input type and epilogue family, and rarely taken paths
//   (unaligned loads, the general four-column epilogue) are out-of-line or separate instantiations:
//   the hot loops of the three roles must stay resident in the instruction cache together.
//
// dw_tc_tma_kernel (weight gradient from the operand caches)
//   Six warps: TMA loads of both MN-major operands (64 slots x 64 columns boxes), tcgen05.mma, four
//   warps draining TMEM.  One work item = (segment of one expert's padded rows, two output tiles);
//   partial tiles are summed in segment order by dw_reduce_kernel: no atomics.
//
// dw_tc_mn_kernel (weight gradient from fp32 / bf16 rows)
//   The stand-alone variant: both operands are gathered, clamped / scaled and converted by 26
//   prologue warps into the same MN-major tiles.
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
// forward / dX kernel geometry: 2 control warps + 22 worker warps whose split between epilogue and
// prologue is chosen per launch (4 ... 20 epilogue warps).  24 warps x 80 registers measured better than 32 x 64
// (which spilled) and than 20 x 102.
constexpr int kWorkerWarps = 22;
constexpr int kFwdThreads = (2 + kWorkerWarps) * 32;      // 768
constexpr int kMaxEpiGroups = 6;
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
constexpr int kMaxProdGroups = 1;
constexpr int kNumBars = 3 * kMaxStages + 4 + 2 * kMaxProdGroups + 2;

// Position in the ring of stages, advanced without integer division.
struct RingPos {
  int s; uint32_t ph; int stages;
  __device__ explicit RingPos(int n) : s(0), ph(0), stages(n) {}
  __device__ __forceinline__ void next() { if (++s == stages) { s = 0; ph ^= 1u; } }
};

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
  int n_epi;   // epilogue warps (multiple of 4)
  int n_prod;  // operand-prologue warps; n_epi + n_prod <= kWorkerWarps
  uint32_t tr_off;  // offset of the epilogue warps' exchange blocks (kTrBytesPerWarp each) in dynamic shared memory
  int a_split, b_split;
  int BN, n_tiles, k_chunks, stages;
  int prod_groups;      // 1, or 2: the prologue warps form two groups that take alternate stages, so that one
                        // group's global-load latency overlaps the other group's arithmetic
  uint32_t tmem_cols, stage_bytes, a_bytes, b_bytes;
  uint32_t cs_off;      // offset of the per-warp column-scale staging area in dynamic shared memory
  int cs_per_warp;      // floats per warp and array in that area
  const int32_t* offsets;
  const void* a; int a_dtype; int64_t a_stride; int64_t a_rows; const int32_t* a_row; int a_div;
  const float* ir; const float* a_absmax; float inp_res; int vec_ok;
  // optional operand cache: split(clamp(a, ir) * cache_scale[a_row[i]]) by padded tile row, [tiles*128, cache_stride]
  __nv_bfloat16* cache_hi; __nv_bfloat16* cache_lo; int64_t cache_stride /* rows of the cache */; const float* cache_scale;
  int a_tma;            // the A operand exists as prepared bf16 tiles (an operand cache written by an earlier kernel):
                        // TMA loads it, there is no prologue and every worker warp runs the epilogue
  int item_mode;        // work item = (row tile, n-tile) instead of a row tile with all its n-tiles (only without a
                        // prologue: the A tile is cheap to load again, and small items fill the last wave better)
  const float* g_absmax;  // fp16 operands, input gradient: device scalar max|A|; A is scaled by a power of two derived
                          // from it before the conversion and the result scaled back (NULL: no scaling)
  EpiParams epi;
};

enum { kDacNone = 0, kDacNorm = 1, kDacQuant = 2 };
// Epilogue families: forward with the vectorised fast path (optional Philox noise / ADC / codes),
// input gradient with the fast path (optional clip mask), and the general four-column routine.
enum { kEpiFwd = 0, kEpiDx = 1, kEpiGeneric = 2 };

// Eight consecutive elements of a row starting at column k (zeros past the row end): the general,
// element-by-element version, kept out of line.
struct F8 { float4 a, b; };
static __device__ __noinline__ F8 load8_slow_call(const void* base, int dtype, int64_t row_off, int k, int K) {
  float t[8];
  for (int i = 0; i < 8; ++i) t[i] = (k + i < K) ? load_elem(base, dtype, row_off + k + i) : 0.f;
  F8 r;
  r.a = make_float4(t[0], t[1], t[2], t[3]);
  r.b = make_float4(t[4], t[5], t[6], t[7]);
  return r;
}
__device__ __forceinline__ void load8_slow(const void* base, int dtype, int64_t row_off, int k, int K, float v[8]) {
  const F8 r = load8_slow_call(base, dtype, row_off, k, K);
  v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}

template <bool F32>
__device__ __forceinline__ void load8_fast(const void* base, int64_t row_off, int k, float v[8]) {
  if (F32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + row_off + k);
    const float4 x = __ldg(q), y = __ldg(q + 1);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
  } else {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + row_off + k));
    v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
    v[4] = __uint_as_float(x.z << 16); v[5] = __uint_as_float(x.z & 0xffff0000u);
    v[6] = __uint_as_float(x.w << 16); v[7] = __uint_as_float(x.w & 0xffff0000u);
  }
}

// Dispatching loader used by the dW prologue (dtype known only at run time).
__device__ __forceinline__ void load8(const void* base, int dtype, int64_t row_off, int k, int K, bool vec_ok,
                                      float v[8]) {
  if (k + 8 <= K && vec_ok) {
    if (dtype == AMOE_F32) load8_fast<true>(base, row_off, k, v);
    else load8_fast<false>(base, row_off, k, v);
  } else {
    load8_slow(base, dtype, row_off, k, K, v);
  }
}

__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Two values -> one packed pair of the operand format (fp16 when F16, else bf16).
template <bool F16>
__device__ __forceinline__ uint32_t cvt_op2(float lo, float hi) {
  if (F16) return cvt_f16x2(lo, hi);
  return cvt_bf16x2(lo, hi);
}

// Eight values -> one 16-byte chunk of the operand format (and, bf16 only, a second chunk with the rounding
// residuals).  tile_hi / tile_lo are shared-memory addresses.
template <bool F16 = false>
__device__ __forceinline__ void store8_rt(uint32_t tile_hi, uint32_t tile_lo, uint32_t off, const float v[8], bool split) {
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = cvt_op2<F16>(v[2 * i], v[2 * i + 1]);
  sts128(tile_hi + off, h[0], h[1], h[2], h[3]);
  if (!F16 && split) {
    uint32_t l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      l[i] = cvt_bf16x2(v[2 * i] - __uint_as_float(h[i] << 16), v[2 * i + 1] - __uint_as_float(h[i] & 0xffff0000u));
    sts128(tile_lo + off, l[0], l[1], l[2], l[3]);
  }
}
template <bool SPLIT>
__device__ __forceinline__ void store8(uint32_t tile_hi, uint32_t tile_lo, uint32_t off, const float v[8]) {
  store8_rt(tile_hi, tile_lo, off, v, SPLIT);
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
  // (pointer arithmetic on the shared array itself, so that accesses through `base` stay shared-memory accesses)
  const uint32_t pad = (1024u - (smem_u32(raw) & 1023u)) & 1023u;
  s.base = raw + pad;
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
    for (int g = 0; g < 2 * kMaxProdGroups; ++g) mbar_init(bar_group(s.bars, g), prod_warps);
    mbar_init(bar_group(s.bars, 2 * kMaxProdGroups), epi_warps);
    mbar_init(bar_group(s.bars, 2 * kMaxProdGroups + 1), epi_warps);
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
  int src;             // source row, or -1 if the row is not to be read
  float ir, rcp_ir;    // input range and its correctly rounded reciprocal
  float am;            // abs-max divisor (its reciprocal is recomputed where it is used: rare mode)
};

// ---- epilogue of one 16-column chunk, fast families (everything 16-byte aligned, n_out % 4 == 0,
// chunk entirely inside the row).
//
// A thread owns one row of the accumulator, so a plain vector store would touch 32 different cache
// lines per instruction.  Instead the warp turns its 32 x 16 block through a private piece of shared
// memory (32 rows of 80 bytes: 64 of data, 16 of padding that keeps both access patterns free of bank
// conflicts): written by row owners, read back so that thread j of a quad holds columns 4j..4j+3 of the
// quad's four rows - every global store then writes 64 contiguous bytes per row, eight rows at a time.
// The clip reference of the input-gradient launches comes the other way through a second such block, filled by
// cp.async one chunk ahead (xref_prefetch).  Eight shared-memory instructions per thread and exchange (a shuffle
// network took 16 shuffles and 48 selects).
// All 32 lanes take part; rows that must not be written carry dst = -1.
constexpr int kTrRowFloats = 20;                          // 80 bytes
constexpr uint32_t kTrBytesPerWarp = 32 * kTrRowFloats * 4;   // 2560

// v = the 16 columns of row `lane`   ->   t[i] = columns 4*(lane&3).. of row (lane & ~3) + i
__device__ __forceinline__ void owner_to_rows(float* tr, const float v[16], float4 t[4], int lane) {
  float* w = tr + lane * kTrRowFloats;
#pragma unroll
  for (int c = 0; c < 4; ++c) *reinterpret_cast<float4*>(w + 4 * c) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
  const float* r = tr + (lane & ~3) * kTrRowFloats + 4 * (lane & 3);
#pragma unroll
  for (int i = 0; i < 4; ++i) t[i] = *reinterpret_cast<const float4*>(r + i * kTrRowFloats);
  __syncwarp();
}

// Rows of the quad this lane belongs to: destination rows (or -1) and clip-reference rows.
struct QuadRows {
  int dst[4];
  int xrow[4];
};

__device__ __forceinline__ void store16_t(const EpiParams& p, const QuadRows& qr, int n0, const float v[16], int lane,
                                          float* tr) {
  if (p.out == nullptr) return;     // codes only (uniform across the kernel)
  float4 t[4];
  owner_to_rows(tr, v, t, lane);
  const int col = n0 + 4 * (lane & 3);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (qr.dst[i] >= 0) {
      const int64_t base = static_cast<int64_t>(qr.dst[i]) * p.out_stride + col;
      if (p.out_dtype == AMOE_F32)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + base) = t[i];
      else
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + base) =
            make_uint2(cvt_bf16x2(t[i].x, t[i].y), cvt_bf16x2(t[i].z, t[i].w));
    }
  }
}

// cs / cis: this chunk's 16 column scales and reciprocals in shared memory (staged by the warp).
// kValue = false: only the ADC codes leave the kernel, the dequantised values are not formed.
// The ADC code rint(x) is taken as (x + 1.5*2^23) - 1.5*2^23 (exact round-to-nearest-even for |x| < 2^22; codes are
// at most 127 in magnitude), whose low mantissa byte is the code in two's complement.
// NOISE / ADC are compile-time copies of the launch's options (the caller dispatches once per chunk): the arithmetic
// runs as packed pairs (two columns per instruction) with the rounding of the scalar definition - every product and
// sum below is one IEEE operation in the order (acc*res + (std*s)*z) * (1/s) -> clamp -> * (1/step) -> round.
template <bool kValue, bool F16, bool NOISE, bool ADC>
__device__ __forceinline__ void epi_chunk_fwd_t(const EpiParams& p, const RowCtx& c, const QuadRows& qr, int n0,
                                                float v[16], const float* cs, const float* cis, int lane, float* tr) {
  constexpr float kMagic = 12582912.f;
  const float post = c.absmax * c.ir;
  const f32x2 accmul2 = pack2(p.acc_mul, p.acc_mul), nstd2 = pack2(p.noise_std, p.noise_std);
  const f32x2 istep2 = pack2(p.adc.inv_step, p.adc.inv_step), step2 = pack2(p.adc.step, p.adc.step);
  const f32x2 magic2 = pack2(kMagic, kMagic), nmagic2 = pack2(-kMagic, -kMagic), post2 = pack2(post, post);
  uint32_t pk[4] = {0u, 0u, 0u, 0u};
  uint4 w = make_uint4(0u, 0u, 0u, 0u);      // one Philox call gives the noise of eight columns: two quads
#pragma unroll
  for (int qd = 0; qd < 4; ++qd) {
    float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 s4 = make_float4(1.f, 1.f, 1.f, 1.f), i4 = s4;
    if (NOISE || ADC) s4 = *reinterpret_cast<const float4*>(cs + 4 * qd);
    if (ADC) i4 = *reinterpret_cast<const float4*>(cis + 4 * qd);
    if (NOISE) {
      if ((qd & 1) == 0)
        w = philox4x32_10_keys(static_cast<uint32_t>(c.dst), static_cast<uint32_t>((n0 >> 3) + (qd >> 1)), kStreamOutNoise,
                               c.noise_offset, p.pkeys);
      box_muller16((qd & 1) ? w.z : w.x, z.x, z.y);
      box_muller16((qd & 1) ? w.w : w.y, z.z, z.w);
    }
    const f32x2 sp[2] = {pack2(s4.x, s4.y), pack2(s4.z, s4.w)}, ip[2] = {pack2(i4.x, i4.y), pack2(i4.z, i4.w)};
    const f32x2 zp[2] = {pack2(z.x, z.y), pack2(z.z, z.w)};
    float tb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      f32x2 acc = mul2(pack2(v[4 * qd + 2 * h], v[4 * qd + 2 * h + 1]), accmul2);
      if (NOISE) acc = add2(acc, mul2(mul2(nstd2, sp[h]), zp[h]));
      if (ADC) {
        float x0, x1;
        unpack2(mul2(acc, ip[h]), x0, x1);
        x0 = fminf(fmaxf(x0, -p.adc.out_bound), p.adc.out_bound);
        x1 = fminf(fmaxf(x1, -p.adc.out_bound), p.adc.out_bound);
        const f32x2 t = add2(mul2(pack2(x0, x1), istep2), magic2);
        unpack2(t, tb[2 * h], tb[2 * h + 1]);
        if (kValue) acc = mul2(mul2(add2(t, nmagic2), step2), sp[h]);
      }
      if (kValue) {
        float y0, y1;
        unpack2(mul2(acc, post2), y0, y1);
        v[4 * qd + 2 * h] = p.out_relu ? fmaxf(y0, 0.f) : y0;
        v[4 * qd + 2 * h + 1] = p.out_relu ? fmaxf(y1, 0.f) : y1;
      }
    }
    if (ADC)
      pk[qd] = __byte_perm(__byte_perm(__float_as_uint(tb[0]), __float_as_uint(tb[1]), 0x0040),
                           __byte_perm(__float_as_uint(tb[2]), __float_as_uint(tb[3]), 0x0040), 0x5410);
  }
  if (p.out_codes && c.valid) {
    // 16 codes of the row; a row starts on a 16-byte boundary only if n_out is a multiple of 16
    int8_t* dstc = p.out_codes + c.dst * p.n_out + n0;
    if ((p.n_out & 15) == 0) {
      *reinterpret_cast<uint4*>(dstc) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    } else {
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) *reinterpret_cast<uint32_t*>(dstc + 4 * qd) = pk[qd];   // n_out % 4 == 0
    }
  }
  if (kValue && (p.next_codes || p.out_cache_hi)) {
    // the row once more as the next projection's operands (padded tile row, [64-column block][row][64]): DAC codes
    // for its forward pass, clamped and scaled bf16 hi (+ lo) terms for its weight gradient
    const int64_t co = (((n0 >> 6) * p.out_cache_stride + c.pad_row) << 6) + (n0 & 63);
    const float rcp_res = quant_rcp(p.next_res);
    const float sc = c.out_cache_sc;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float hc[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        float t = c.valid ? v[8 * half + x] : 0.f;
        if (p.out_dtype == AMOE_BF16) t = __bfloat162float(__float2bfloat16_rn(t));   // what the next kernel would read
        hc[x] = p.next_ir ? clamp_ir(t, c.next_ir) : t;
      }
      if (p.next_codes) {
        uint32_t q[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          // rint((h / ir) / res) with IEEE-exact quotients, as packed pairs (dac_code_clamped, two at a time)
          f32x2 t = div_by_rcp2(pack2(hc[2 * x], hc[2 * x + 1]), pack2(-c.next_ir, -c.next_ir), pack2(c.next_rcp, c.next_rcp));
          t = div_by_rcp2(t, pack2(-p.next_res, -p.next_res), pack2(rcp_res, rcp_res));
          t = add2(add2(t, pack2(12582912.f, 12582912.f)), pack2(-12582912.f, -12582912.f));
          float q0, q1;
          unpack2(t, q0, q1);
          q[x] = cvt_op2<F16>(q0, q1);
        }
        *reinterpret_cast<uint4*>(p.next_codes + co + 8 * half) = make_uint4(q[0], q[1], q[2], q[3]);
      }
      if (p.out_cache_hi) {
        uint32_t h[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) h[x] = cvt_op2<F16>(hc[2 * x] * sc, hc[2 * x + 1] * sc);
        *reinterpret_cast<uint4*>(p.out_cache_hi + co + 8 * half) = make_uint4(h[0], h[1], h[2], h[3]);
        if (!F16 && p.out_cache_lo) {
          uint32_t l[4];
#pragma unroll
          for (int x = 0; x < 4; ++x)
            l[x] = cvt_bf16x2(hc[2 * x] * sc - __uint_as_float(h[x] << 16), hc[2 * x + 1] * sc - __uint_as_float(h[x] & 0xffff0000u));
          *reinterpret_cast<uint4*>(p.out_cache_lo + co + 8 * half) = make_uint4(l[0], l[1], l[2], l[3]);
        }
      }
    }
  }
  if (kValue) store16_t(p, qr, n0, v, lane, tr);
}

template <bool kValue, bool F16>
__device__ __forceinline__ void epi_chunk_fwd(const EpiParams& p, const RowCtx& c, const QuadRows& qr, int n0,
                                              float v[16], const float* cs, const float* cis, int lane, float* tr) {
  const bool noise = p.noise_std > 0.f, adc = p.adc.on;
  if (noise && adc) epi_chunk_fwd_t<kValue, F16, true, true>(p, c, qr, n0, v, cs, cis, lane, tr);
  else if (adc) epi_chunk_fwd_t<kValue, F16, false, true>(p, c, qr, n0, v, cs, cis, lane, tr);
  else if (noise) epi_chunk_fwd_t<kValue, F16, true, false>(p, c, qr, n0, v, cs, cis, lane, tr);
  else epi_chunk_fwd_t<kValue, F16, false, false>(p, c, qr, n0, v, cs, cis, lane, tr);
}

// `cache_mul`: the operand cache keeps the result times this power of two (the gradient scale of fp16 operands).
// Clip-reference rows of one 16-column chunk, asynchronously into the warp's reference block: lane l copies columns
// 4*(l&3).. of the quad's rows (l & ~3) + i, 16 bytes each for fp32 (8 for bf16), zero-filled for rows that are not
// read.  Issued one chunk ahead, so that the latency of these gathered loads overlaps the previous chunk's arithmetic.
__device__ __forceinline__ void xref_prefetch(const EpiParams& p, const QuadRows& qr, int n0, float* xb, int lane) {
  const int col = n0 + 4 * (lane & 3);
  float* w = xb + (lane & ~3) * kTrRowFloats + 4 * (lane & 3);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool on = qr.xrow[i] >= 0;
    const int64_t xi = on ? static_cast<int64_t>(qr.xrow[i]) * p.x_ref_stride + col : 0;
    const uint32_t dst = smem_u32(w + i * kTrRowFloats);
    if (p.x_ref_dtype == AMOE_F32) cp_async16(dst, reinterpret_cast<const float*>(p.x_ref) + xi, on ? 16u : 0u);
    else cp_async8(dst, reinterpret_cast<const __nv_bfloat16*>(p.x_ref) + xi, on ? 8u : 0u);
  }
  cp_async_commit();
}

// XREF / IR / RELU / CACHE are compile-time copies of the launch's options (x_ref given, input ranges given, ReLU
// mask, result rows also written as an operand cache); the caller dispatches once per chunk.
template <bool F16, bool XREF, bool IR, bool RELU, bool CACHE>
__device__ __forceinline__ void epi_chunk_dx_t(const EpiParams& p, RowCtx& c, const QuadRows& qr, int n0, float v[16],
                                               int lane, float cache_mul, float* tr, float* xb, int next_n0) {
  if (XREF) {
    // this chunk's reference rows were requested one chunk ago (xref_prefetch): wait for them, take "my row, 16
    // columns" out of the block, then request the next chunk's before the arithmetic starts
    float xr[16];
    cp_async_wait<0>();
    __syncwarp();
    const float* rp = xb + lane * kTrRowFloats;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const float4 u = *reinterpret_cast<const float4*>(rp + 4 * cc);
      if (p.x_ref_dtype == AMOE_F32) {
        xr[4 * cc] = u.x; xr[4 * cc + 1] = u.y; xr[4 * cc + 2] = u.z; xr[4 * cc + 3] = u.w;
      } else {      // four bf16 in the first eight bytes
        const uint32_t a = __float_as_uint(u.x), b = __float_as_uint(u.y);
        xr[4 * cc] = __uint_as_float(a << 16); xr[4 * cc + 1] = __uint_as_float(a & 0xffff0000u);
        xr[4 * cc + 2] = __uint_as_float(b << 16); xr[4 * cc + 3] = __uint_as_float(b & 0xffff0000u);
      }
    }
    __syncwarp();
    if (next_n0 >= 0) xref_prefetch(p, qr, next_n0, xb, lane);
    if (IR) {
      // up = x >= ir adds min(g, 0), low = x <= -ir subtracts max(g, 0), everything else is kept (cvmm.py:863-870).
      // With t = g carrying x's sign flipped in (exact), both clipped cases are min(t, 0): one compare, one min.
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float gs = v[j] * c.rs;
        const bool keep = fabsf(xr[j]) < c.ir;
        const float tj = __uint_as_float(__float_as_uint(gs) ^ (__float_as_uint(xr[j]) & 0x80000000u));
        const bool clipped = fabsf(xr[j]) >= c.ir;      // (false for a NaN reference, like `up` and `low`)
        if (clipped) c.dir_acc += fminf(tj, 0.f);
        c.keep += keep ? 1u : 0u;
        v[j] = keep ? gs : 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= c.rs;
    }
    if (RELU) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = xr[j] > 0.f ? v[j] : 0.f;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] *= c.rs;
  }
  if (CACHE) {
    // the row once more as bf16 hi (+ lo) terms at its padded tile row: the B operand of the next dW
    // layout [64-column block][padded row][64]; n0 is a multiple of 16, so the chunk stays inside one block
    const int64_t co = (((n0 >> 6) * p.out_cache_stride + c.pad_row) << 6) + (n0 & 63);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t h[4];
#pragma unroll
      for (int x = 0; x < 4; ++x)
        h[x] = c.valid ? cvt_op2<F16>(v[8 * half + 2 * x] * cache_mul, v[8 * half + 2 * x + 1] * cache_mul) : 0u;
      *reinterpret_cast<uint4*>(p.out_cache_hi + co + 8 * half) = make_uint4(h[0], h[1], h[2], h[3]);
      if (!F16 && p.out_cache_lo) {
        uint32_t l[4];
#pragma unroll
        for (int x = 0; x < 4; ++x)
          l[x] = c.valid ? cvt_bf16x2(v[8 * half + 2 * x] - __uint_as_float(h[x] << 16),
                                      v[8 * half + 2 * x + 1] - __uint_as_float(h[x] & 0xffff0000u)) : 0u;
        *reinterpret_cast<uint4*>(p.out_cache_lo + co + 8 * half) = make_uint4(l[0], l[1], l[2], l[3]);
      }
    }
  }
  store16_t(p, qr, n0, v, lane, tr);
}

template <bool F16>
__device__ __forceinline__ void epi_chunk_dx(const EpiParams& p, RowCtx& c, const QuadRows& qr, int n0, float v[16],
                                             int lane, float cache_mul, float* tr, float* xb, int next_n0) {
  const bool xref = p.x_ref != nullptr, ir = xref && p.ir != nullptr, relu = xref && p.x_ref_relu != 0;
  const bool cache = p.out_cache_hi != nullptr;
  // the two launches of a layer step, then the remaining combinations
  if (xref && ir && relu && cache) epi_chunk_dx_t<F16, true, true, true, true>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (xref && ir && !relu && !cache) epi_chunk_dx_t<F16, true, true, false, false>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (!xref && !cache) epi_chunk_dx_t<F16, false, false, false, false>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (!xref) epi_chunk_dx_t<F16, false, false, false, true>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (ir && relu) epi_chunk_dx_t<F16, true, true, true, false>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (ir) epi_chunk_dx_t<F16, true, true, false, true>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
  else if (cache) epi_chunk_dx_t<F16, true, false, true, true>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);   // x_ref without ir: ReLU mask only
  else epi_chunk_dx_t<F16, true, false, true, false>(p, c, qr, n0, v, lane, cache_mul, tr, xb, next_n0);
}

// Work items of one CTA: row tile t with all its n-tiles, or - item mode - one (row tile, n-tile) pair.
struct ItemWalk {
  TileIter ti;
  int n_tiles, item_mode;
  int64_t w;
  int e, row0, rows, nt0, nt1;
  int64_t t;
  __device__ ItemWalk(const TcParams& p) : ti(p.offsets, p.E), n_tiles(p.n_tiles), item_mode(p.item_mode), w(blockIdx.x) {}
  __device__ bool get() {
    t = item_mode ? w / n_tiles : w;
    if (!ti.get(t, e, row0, rows)) return false;
    nt0 = item_mode ? static_cast<int>(w - t * n_tiles) : 0;
    nt1 = item_mode ? nt0 + 1 : n_tiles;
    return true;
  }
  __device__ void next() { w += gridDim.x; }
};

template <int DAC, bool A_F32, int EPI, bool F16>
__global__ void __launch_bounds__(kFwdThreads, 1)
cvmm_tc_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo,
               const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo, TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ RowMeta s_meta[kMaxProdGroups][kBM];
  __shared__ float s_cscale[kBM];
  __shared__ float s_dir[kMaxEpiGroups][kBM];
  __shared__ unsigned s_keep[kMaxEpiGroups][kBM];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_prod = p.a_tma ? 0 : p.n_prod;
  setup_cta(sm, p.stages, p.tmem_cols, n_prod > 0 ? n_prod / p.prod_groups : 1, p.n_epi, n_prod > 0 ? n_prod : 1, p.n_epi);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.epi.status;
  // gradient scale of fp16 operands (input gradient only): a power of two from the tensor's largest magnitude
  float g_mul = 1.f, g_inv = 1.f;
  if (F16 && p.g_absmax != nullptr) g_mul = grad_pow2_scale(__ldg(p.g_absmax), g_inv);

  if (warp == 0) {
    // ---------------------------------------------------------------- weight tiles by TMA
    if (lane == 0) {
      tma_prefetch_desc(&tmap_hi);
      if (p.b_split) tma_prefetch_desc(&tmap_lo);
      if (p.a_tma) { tma_prefetch_desc(&tmap_a_hi); if (p.a_split) tma_prefetch_desc(&tmap_a_lo); }
      RingPos rp(p.stages);
      bool alive = true;
      for (ItemWalk it(p); alive && it.get(); it.next()) {
        for (int nt = it.nt0; nt < it.nt1 && alive; ++nt) {
          for (int kc = 0; kc < p.k_chunks; ++kc, rp.next()) {
            const int s = rp.s;
            const uint32_t ph = rp.ph;
            if (!mbar_wait(bar_empty(sm.bars, s), ph ^ 1u, sm.abort_flag, status, 1, 64)) { alive = false; break; }
            const uint32_t dst = sm.base_u32 + s * p.stage_bytes + p.a_bytes;
            mbar_arrive_expect_tx(bar_full_b(sm.bars, s), p.b_bytes * (p.b_split ? 2u : 1u) + (p.a_tma ? p.a_bytes : 0u));
            if (p.a_tma) {
              // A tile: 128 padded tile rows x 64 columns of block kc of the cache (K-major, 128-byte swizzle)
              const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
              tma_load_3d(sa, &tmap_a_hi, bar_full_b(sm.bars, s), 0, static_cast<int>(it.t * kBM), kc);
              if (p.a_split) tma_load_3d(sa + kATile, &tmap_a_lo, bar_full_b(sm.bars, s), 0, static_cast<int>(it.t * kBM), kc);
            }
            tma_load_3d(dst, &tmap_hi, bar_full_b(sm.bars, s), kc * kBK, nt * p.BN, it.e);
            if (p.b_split) tma_load_3d(dst + p.b_bytes, &tmap_lo, bar_full_b(sm.bars, s), kc * kBK, nt * p.BN, it.e);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc = F16 ? make_idesc_f16(kBM, p.BN) : make_idesc_bf16(kBM, p.BN);
      RingPos rp(p.stages);
      uint32_t acc_it = 0;
      bool alive = true;
      for (ItemWalk it(p); alive && it.get(); it.next()) {
        for (int nt = it.nt0; nt < it.nt1 && alive; ++nt, ++acc_it) {
          const int buf = acc_it & 1u;
          const uint32_t aph = (acc_it >> 1) & 1u;
          if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 2)) { alive = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * p.BN);
          for (int kc = 0; kc < p.k_chunks; ++kc, rp.next()) {
            const int s = rp.s;
            const uint32_t ph = rp.ph;
            if (!p.a_tma && !mbar_wait(bar_full_a(sm.bars, s), ph, sm.abort_flag, status, 3)) { alive = false; break; }
            if (!mbar_wait(bar_full_b(sm.bars, s), ph, sm.abort_flag, status, 4)) { alive = false; break; }
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
              if (p.b_split) umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
              if (p.a_split) umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
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
    const int r = q * 32 + lane;
    constexpr int cw = 16;                     // chunk width in columns
    const int chunks = p.BN / cw;
    float* cs_smem = reinterpret_cast<float*>(sm.base + p.cs_off) + ew * 2 * p.cs_per_warp;
    float* cis_smem = cs_smem + p.cs_per_warp;
    float* tr = reinterpret_cast<float*>(sm.base + p.tr_off) + ew * (kTrBytesPerWarp / 4);   // this warp's exchange block
    // a second block per warp receives the clip-reference rows one chunk ahead (input-gradient launches with x_ref)
    float* xb = tr + p.n_epi * (kTrBytesPerWarp / 4);
    const bool xpre = EPI == kEpiDx && p.epi.x_ref != nullptr;
    const bool need_cs = EPI == kEpiFwd && (p.epi.noise_std > 0.f || p.epi.adc.on);
    uint32_t acc_it = 0, sync_round = 0;
    bool alive = true;
    for (ItemWalk it(p); alive && it.get(); it.next()) {
      const int e = it.e, rows = it.rows;
      const int64_t t = it.t;
      const int64_t i = static_cast<int64_t>(it.row0) + r;
      RowCtx ctx = epi_row_begin(p.epi, i, e, r < rows);
      ctx.pad_row = t * kBM + r;
      if (EPI == kEpiFwd && p.epi.out_cache_hi && p.epi.out_cache_scale && ctx.valid)
        ctx.out_cache_sc = p.epi.out_cache_scale[ctx.dst];      // once per tile, not once per chunk
      // the accumulator carries the gradient scale of the A operand: take it out with the row scale
      if (EPI != kEpiFwd && p.epi.is_dx) ctx.rs *= g_inv;
      if (grp == 0 && it.nt0 == 0) epi_row_side_outputs(p.epi, ctx);
      QuadRows qr;
      if (EPI != kEpiGeneric) {
        const int my_dst = ctx.valid ? static_cast<int>(ctx.dst) : -1;
        const int my_x = (ctx.valid && p.epi.is_dx && p.epi.x_ref) ? static_cast<int>(ctx.xrow) : -1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          qr.dst[j] = __shfl_sync(0xffffffffu, my_dst, (lane & ~3) + j);
          qr.xrow[j] = __shfl_sync(0xffffffffu, my_x, (lane & ~3) + j);
        }
      }
      if (xpre && grp < chunks && it.nt0 * p.BN + grp * cw + cw <= p.epi.n_out)
        xref_prefetch(p.epi, qr, it.nt0 * p.BN + grp * cw, xb, lane);     // the item's first chunk, before its accumulator is ready
      for (int nt = it.nt0; nt < it.nt1 && alive; ++nt, ++acc_it) {
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (need_cs) {
          // this warp's chunks of col_scale / col_inv_scale, staged while the MMAs are still running
          __syncwarp();
          int slot = 0;
          for (int ch = grp; ch < chunks; ch += groups, ++slot) {
            const int n = nt * p.BN + ch * cw + (lane & (cw - 1));
            if (n < p.epi.n_out) {
              const int64_t ci = static_cast<int64_t>(e) * p.epi.n_out + n;
              if (lane < cw) cs_smem[slot * cw + lane] = p.epi.col_scale[ci];
              else if (lane >= 16 && lane < 16 + cw && p.epi.adc.on) cis_smem[slot * cw + lane - 16] = p.epi.col_inv_scale[ci];
            }
          }
          __syncwarp();
        }
        bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 5, 128);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * p.BN);
        int slot = 0;
#pragma unroll 1
        for (int ch = grp; ch < chunks; ch += groups, ++slot) {
          float v[16];
          tmem_ld16(taddr + ch * 16, v);
          tmem_ld_wait();
          const int n0 = nt * p.BN + ch * 16;
          if (EPI == kEpiGeneric || n0 + 16 > p.epi.n_out) {
#pragma unroll 1
            for (int qd = 0; qd < 4; ++qd) {
              const float w4[4] = {v[0], v[1], v[2], v[3]};
              epi_quad(p.epi, ctx, n0 + 4 * qd, w4);
#pragma unroll
              for (int j = 0; j < 12; ++j) v[j] = v[j + 4];   // rotate the next four columns in
            }
          } else {   // all 32 lanes: the quad exchange needs every lane, invalid rows are masked inside
            if (EPI == kEpiFwd) {
              if (p.epi.out != nullptr) epi_chunk_fwd<true, F16>(p.epi, ctx, qr, n0, v, cs_smem + slot * 16, cis_smem + slot * 16, lane, tr);
              else epi_chunk_fwd<false, F16>(p.epi, ctx, qr, n0, v, cs_smem + slot * 16, cis_smem + slot * 16, lane, tr);
            }
            else {
              // the chunk this warp takes next (same n-tile, or the first of the next n-tile), if it is a whole one
              int next_n0 = -1;
              if (xpre) {
                if (ch + groups < chunks) next_n0 = n0 + groups * cw;
                else if (nt + 1 < it.nt1) next_n0 = (nt + 1) * p.BN + grp * cw;
                if (next_n0 + cw > p.epi.n_out) next_n0 = -1;
              }
              epi_chunk_dx<F16>(p.epi, ctx, qr, n0, v, lane, g_mul, tr, xb, next_n0);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      }
      if (!alive) break;
      if (p.epi.is_dx && (p.epi.ir_grad || p.epi.keep_count)) {
        // fixed-order combination of the groups' partial row sums (an item holds all n-tiles of its rows here:
        // item mode is never combined with these per-row results)
        if (groups > 1) {
          s_dir[grp][r] = ctx.dir_acc;
          s_keep[grp][r] = ctx.valid ? ctx.keep : 0u;
          if (!group_sync(bar_group(sm.bars, 2 * kMaxProdGroups), sync_round, sm.abort_flag, status, 7)) { alive = false; break; }
          if (grp == 0) {
            float d = s_dir[0][r];
            unsigned kc = s_keep[0][r];
            for (int g = 1; g < groups; ++g) { d += s_dir[g][r]; kc += s_keep[g][r]; }
            ctx.dir_acc = d;
            ctx.keep = kc;
          }
          if (!group_sync(bar_group(sm.bars, 2 * kMaxProdGroups + 1), sync_round, sm.abort_flag, status, 8)) { alive = false; break; }
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
  } else if (!p.a_tma && warp < 2 + p.n_epi + n_prod) {
    // ---------------------------------------------------------------- operand prologue (A tiles from rows)
    const int np_all = n_prod * 32;
    const int pt_all = threadIdx.x - (2 + p.n_epi) * 32;  // 0..np_all-1
    const int pw = warp - (2 + p.n_epi);
    const bool two = p.prod_groups == 2;
    const uint32_t grp = two ? static_cast<uint32_t>(pw & 1) : 0u;
    const int np = two ? (n_prod >> 1) * 32 : np_all;      // threads that share one stage
    const int pt = two ? (pw >> 1) * 32 + lane : pt_all;
    const bool has_ir = DAC != kDacNone && p.ir != nullptr, has_am = DAC != kDacNone && p.a_absmax != nullptr;
    const bool a_split = p.a_split != 0;
    const float rcp_res = quant_rcp(p.inp_res);
    RowMeta* meta = s_meta[0];
    TileIter ti(p.offsets, p.E);
    RingPos rp(p.stages);
    uint32_t it = 0, sync_round = 0;
    bool alive = true;
    for (int64_t t = blockIdx.x; alive; t += gridDim.x) {
      int e, row0, rows;
      if (!ti.get(t, e, row0, rows)) break;
      // everyone is done with the previous tile's metadata
      if (!group_sync(bar_group(sm.bars, 0), sync_round, sm.abort_flag, status, 9)) break;
      for (int r = pt_all; r < kBM; r += np_all) {
        RowMeta m;
        m.src = -1; m.ir = 1.f; m.rcp_ir = 1.f; m.am = 1.f;
        float csc = 0.f;
        if (r < rows) {
          const int64_t i = static_cast<int64_t>(row0) + r;
          const int64_t raw = p.a_row[i];
          const int64_t src = raw / p.a_div;
          if (p.cache_scale && src >= 0 && src < p.a_rows) csc = p.cache_scale[raw];
          if (src < 0 || src >= p.a_rows) {
            report(status, AMOE_ERR_INDEX_RANGE, 20, static_cast<int>(i), static_cast<int>(src));
          } else {
            m.src = static_cast<int>(src);
            if (has_ir) { m.ir = p.ir[p.epi.ir_by_expert ? e : i]; m.rcp_ir = __frcp_rn(m.ir); }
            if (has_am) m.am = p.a_absmax[src];
          }
        }
        meta[r] = m;
        if (p.cache_scale) s_cscale[r] = csc;
      }
      if (!group_sync(bar_group(sm.bars, 1), sync_round, sm.abort_flag, status, 10)) break;
      ++sync_round;
      for (int nt = 0; nt < p.n_tiles && alive; ++nt) {
        const bool do_cache = p.cache_hi != nullptr && nt == 0;
        for (int kc = 0; kc < p.k_chunks; ++kc, ++it, rp.next()) {
          if (two && (it & 1u) != grp) continue;
          const int s = rp.s;
          bool ok = mbar_wait(bar_empty(sm.bars, s), rp.ph ^ 1u, sm.abort_flag, status, 6);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) { alive = false; break; }
          const uint32_t a_hi = sm.base_u32 + s * p.stage_bytes;
          const uint32_t a_lo = a_hi + kATile;
          const bool full_k = (kc + 1) * kBK <= p.Kc && p.vec_ok;
          // 1024 tasks (128 rows x 8 sixteen-byte chunks), two per thread and round
#pragma unroll 1
          for (int base = pt; base < kBM * 8; base += np * 2) {
            float v[2][8];
            RowMeta m[2];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const int task = base + b * np;
              m[b].src = -1;
              if (task < kBM * 8) m[b] = meta[task >> 3];
              const int k = kc * kBK + (task & 7) * 8;
              const int64_t off = static_cast<int64_t>(m[b].src) * p.a_stride;
              if (m[b].src >= 0 && full_k) {
                load8_fast<A_F32>(p.a, off, k, v[b]);
              } else if (m[b].src >= 0 && k < p.Kc) {
                load8_slow(p.a, p.a_dtype, off, k, p.Kc, v[b]);
              } else {
                m[b].src = -1;
#pragma unroll
                for (int x = 0; x < 8; ++x) v[b][x] = 0.f;
              }
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const int task = base + b * np;
              if (task < kBM * 8) {
                const int kk = kc * kBK + (task & 7) * 8;
                const bool cache_now = do_cache && kk < p.Kc;
                // cache layout: [64-column block][padded row][64]
                const int64_t co = cache_now ? ((kc * p.cache_stride + t * kBM + (task >> 3)) << 6) + (task & 7) * 8 : 0;
                const uint32_t soff = sw128_offset(task >> 3, task & 7);
                if (DAC == kDacNone) {
                  if (F16) {
#pragma unroll
                    for (int x = 0; x < 8; ++x) v[b][x] *= g_mul;
                  }
                  // the tile and the cache hold the same terms: convert once, store twice
                  uint32_t h[4], l[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                  for (int x = 0; x < 4; ++x) h[x] = cvt_op2<F16>(v[b][2 * x], v[b][2 * x + 1]);
                  if (!F16 && (a_split || (cache_now && p.cache_lo))) {
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                      l[x] = cvt_bf16x2(v[b][2 * x] - __uint_as_float(h[x] << 16),
                                        v[b][2 * x + 1] - __uint_as_float(h[x] & 0xffff0000u));
                  }
                  sts128(a_hi + soff, h[0], h[1], h[2], h[3]);
                  if (!F16 && a_split) sts128(a_lo + soff, l[0], l[1], l[2], l[3]);
                  if (cache_now) {
                    *reinterpret_cast<uint4*>(p.cache_hi + co) = make_uint4(h[0], h[1], h[2], h[3]);
                    if (!F16 && p.cache_lo) *reinterpret_cast<uint4*>(p.cache_lo + co) = make_uint4(l[0], l[1], l[2], l[3]);
                  }
                } else {
                  if (has_ir && m[b].src >= 0) {
#pragma unroll
                    for (int x = 0; x < 8; ++x) v[b][x] = clamp_ir(v[b][x], m[b].ir);
                  }
                  if (cache_now) {
                    // the operand as dW wants it: clamped (not quantised), times the per-row scale, hi (+ lo) terms
                    float c8[8];
                    const float sc = p.cache_scale ? s_cscale[task >> 3] : 1.f;
#pragma unroll
                    for (int x = 0; x < 8; ++x) c8[x] = p.cache_scale ? v[b][x] * sc : v[b][x];
                    uint32_t h[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) h[x] = cvt_op2<F16>(c8[2 * x], c8[2 * x + 1]);
                    *reinterpret_cast<uint4*>(p.cache_hi + co) = make_uint4(h[0], h[1], h[2], h[3]);
                    if (!F16 && p.cache_lo) {
                      uint32_t l[4];
#pragma unroll
                      for (int x = 0; x < 4; ++x)
                        l[x] = cvt_bf16x2(c8[2 * x] - __uint_as_float(h[x] << 16), c8[2 * x + 1] - __uint_as_float(h[x] & 0xffff0000u));
                      *reinterpret_cast<uint4*>(p.cache_lo + co) = make_uint4(l[0], l[1], l[2], l[3]);
                    }
                  }
                  if (m[b].src >= 0) {
                    const float rcp_am = has_am ? __frcp_rn(m[b].am) : 1.f;
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                      if (DAC == kDacQuant)
                        v[b][x] = dac_code_clamped(v[b][x], has_ir, m[b].ir, m[b].rcp_ir, has_am, m[b].am, rcp_am, p.inp_res, rcp_res);
                      else
                        v[b][x] = dac_normalise_clamped(v[b][x], has_ir, m[b].ir, m[b].rcp_ir, has_am, m[b].am, rcp_am);
                    }
                  }
                  store8_rt<F16>(a_hi, a_lo, soff, v[b], a_split);
                }
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

// ---------------------------------------------------------------------------- dW, MN-major operands
// The contraction index of dW is the slot, which is the slow index of both row-major inputs.  The
// tensor core takes such operands directly ("MN-major"): a stage holds 64 slots as 64 rows of 128 bytes
// per block of 64 columns, so the prologue converts and stores 16-byte chunks without transposing.
struct DwMnParams {
  int E, K, N;
  int BN, m_tiles, n_tiles, stages;
  int MB, NB;           // a work item owns MB x NB (= 1x1, 2x1 or 1x2) output tiles that share operand tiles
  int seg;              // slots per work segment (multiple of 64); 0: one segment per expert
  uint32_t tmem_cols, stage_bytes, a_bytes, b_bytes;   // a_bytes/b_bytes: one precision term of A / B
  const int32_t* offsets;
  const void* x; int x_dtype; int64_t x_stride; int64_t x_rows; const int32_t* x_row; const float* ir; int ir_by_expert;
  const void* g; int g_dtype; int64_t g_stride; int64_t g_rows; const int32_t* g_row; int g_div;
  const float* g_scale;
  int x_vec_ok, g_vec_ok;
  float* dw;            // [E,K,N]
  float* partials;      // [segments,K,N] when the slot range of an expert is split, else NULL
  int32_t* status;
  int f16;              // fp16 operands (one term)
  const float* g_absmax;  // fp16: device scalar max|g|; g is scaled by the power of two derived from it, dW scaled back
};

constexpr int kDwProdWarps = 26;
constexpr int kDwThreads = (6 + kDwProdWarps) * 32;   // 2 control + 4 epilogue + 26 prologue warps
constexpr uint32_t kMnBlock = kBK * 128;   // 64 rows x 128 bytes

// Segment number `idx` of the slot list: expert e owns ceil(count_e / seg) segments (seg == 0: exactly
// one segment per expert, possibly empty).
struct SegIter {
  const int32_t* off; int E, seg; int e; int64_t before;
  __device__ SegIter(const int32_t* o, int E_, int seg_) : off(o), E(E_), seg(seg_), e(0), before(0) {}
  __device__ bool get(int64_t idx, int& ex, int& beg, int& end) {
    while (e < E) {
      const int b = off[e], en = off[e + 1];
      const int ns = seg > 0 ? (en - b + seg - 1) / seg : 1;
      if (idx < before + ns) {
        ex = e;
        beg = seg > 0 ? b + static_cast<int>(idx - before) * seg : b;
        end = seg > 0 ? min(beg + seg, en) : en;
        return true;
      }
      before += ns;
      ++e;
    }
    return false;
  }
};

// IN: 0 = x and g fp32 with 16-byte aligned rows, 1 = both bf16 aligned, 2 = anything (run-time dispatch)
//
// A work item = (slot segment, block of MB x NB output tiles).  With two tiles per item the operand
// tile they share is converted once instead of twice (the prologue, not the tensor pipe, bounds this
// kernel).  Stage layout: MB A-tiles (hi, lo) then NB B-tiles (hi, lo); TMEM: two buffers of MB*NB
// accumulators.
template <bool SPLIT, int IN>
__global__ void __launch_bounds__(kDwThreads, 1) dw_tc_mn_kernel(DwMnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup_cta(sm, p.stages, p.tmem_cols, kDwProdWarps, 4);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.status;
  const int mb_tiles = (p.m_tiles + p.MB - 1) / p.MB, nb_tiles = (p.n_tiles + p.NB - 1) / p.NB;
  const int tps = mb_tiles * nb_tiles;          // tile blocks per segment
  const int n_acc = p.MB * p.NB;
  const uint32_t a_tile = (SPLIT ? 2u : 1u) * p.a_bytes;   // one A tile, all precision terms
  const uint32_t b_tile = (SPLIT ? 2u : 1u) * p.b_bytes;
  const uint32_t b_region = static_cast<uint32_t>(p.MB) * a_tile;
  float g_mul = 1.f, g_inv = 1.f;       // gradient scale of fp16 operands; a direct store takes it out again,
  if (p.f16 && p.g_absmax != nullptr) g_mul = grad_pow2_scale(__ldg(p.g_absmax), g_inv);
  const float out_mul = p.partials ? 1.f : g_inv;   // partial tiles keep it until dw_reduce_kernel

  if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = p.f16 ? (make_idesc_f16(kBM, p.BN) | (1u << 15) | (1u << 16)) : make_idesc_bf16_mn(kBM, p.BN);
      RingPos rp(p.stages);
      SegIter si(p.offsets, p.E, p.seg);
      uint32_t acc_it = 0;
      bool alive = true;
      for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
        int e, beg, end;
        if (!si.get(w / tps, e, beg, end)) break;
        const int chunks = (end - beg + kBK - 1) / kBK;
        if (chunks == 0) continue;
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 12)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_base = tmem_base + static_cast<uint32_t>(buf * n_acc * p.BN);
        for (int kc = 0; kc < chunks; ++kc, rp.next()) {
          const int s = rp.s;
          if (!mbar_wait(bar_full_a(sm.bars, s), rp.ph, sm.abort_flag, status, 13)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
          for (int acc = 0; acc < n_acc; ++acc) {
            const int ma = acc / p.NB, nb = acc - ma * p.NB;
            const uint32_t at = sa + ma * a_tile, bt = sa + b_region + nb * b_tile;
            const uint64_t da_hi = make_smem_desc_mn_sw128(at, kMnBlock);
            const uint64_t da_lo = make_smem_desc_mn_sw128(at + p.a_bytes, kMnBlock);
            const uint64_t db_hi = make_smem_desc_mn_sw128(bt, kMnBlock);
            const uint64_t db_lo = make_smem_desc_mn_sw128(bt + p.b_bytes, kMnBlock);
            const uint32_t d_tmem = d_base + static_cast<uint32_t>(acc * p.BN);
#pragma unroll
            for (int k16 = 0; k16 < kBK / 16; ++k16) {
              const uint64_t adv = static_cast<uint64_t>(k16 * (16 * 128 / 16));  // 16 rows of 128 bytes, >> 4
              umma_bf16(d_tmem, da_hi + adv, db_hi + adv, idesc, (kc | k16) != 0 ? 1u : 0u);
              if (SPLIT) {
                umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
                umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
              }
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
    SegIter si(p.offsets, p.E, p.seg);
    uint32_t acc_it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
      int e, beg, end;
      const int64_t seg_idx = w / tps;
      if (!si.get(seg_idx, e, beg, end)) break;
      const int sub = static_cast<int>(w - seg_idx * tps);
      const int nbk = sub % nb_tiles, mbk = sub / nb_tiles;
      const int chunks = (end - beg + kBK - 1) / kBK;
      float* out_base = p.partials ? p.partials + seg_idx * p.K * p.N : p.dw + static_cast<int64_t>(e) * p.K * p.N;
      if (chunks == 0) {   // only without segment splitting: an expert nobody was routed to
        for (int acc = 0; acc < n_acc; ++acc) {
          const int ma = acc / p.NB, nb = acc - ma * p.NB;
          const int m = (mbk * p.MB + ma) * kBM + r, n0 = (nbk * p.NB + nb) * p.BN;
          if (m < p.K)
            for (int n = n0; n < min(n0 + p.BN, p.N); ++n) out_base[static_cast<int64_t>(m) * p.N + n] = 0.f;
        }
        continue;
      }
      const int buf = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 15, 128);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      for (int acc = 0; acc < n_acc; ++acc) {
        const int ma = acc / p.NB, nb = acc - ma * p.NB;
        const int m = (mbk * p.MB + ma) * kBM + r, n0 = (nbk * p.NB + nb) * p.BN;
        float* dst = out_base + static_cast<int64_t>(m) * p.N;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               static_cast<uint32_t>((buf * n_acc + acc) * p.BN);
#pragma unroll 1
        for (int c0 = 0; c0 < p.BN; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 16; ++x) v[x] *= out_mul;
          const int n = n0 + c0;
          if (m < p.K && n < p.N) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      ++acc_it;
    }
  } else if (warp >= 6) {
    constexpr int np = kDwProdWarps * 32;
    const int pt = threadIdx.x - 6 * 32;
    constexpr int a_tile_tasks = kBK * (kBM / 8);        // 64 slots x 16 sixteen-byte chunks per A tile
    const int b_chunks = (p.BN + 7) / 8;
    const int b_shift = (b_chunks & (b_chunks - 1)) == 0 ? __ffs(b_chunks) - 1 : -1;
    const int b_tile_tasks = kBK * b_chunks;
    const int a_tasks = p.MB * a_tile_tasks;
    const int tasks = a_tasks + p.NB * b_tile_tasks;
    RingPos rp(p.stages);
    SegIter si(p.offsets, p.E, p.seg);
    bool alive = true;
    for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
      int e, beg, end;
      const int64_t seg_idx = w / tps;
      if (!si.get(seg_idx, e, beg, end)) break;
      const int sub = static_cast<int>(w - seg_idx * tps);
      const int nbk = sub % nb_tiles, mbk = sub / nb_tiles;
      const int chunks = (end - beg + kBK - 1) / kBK;
      for (int kc = 0; kc < chunks; ++kc, rp.next()) {
        const int s = rp.s;
        bool ok = mbar_wait(bar_empty(sm.bars, s), rp.ph ^ 1u, sm.abort_flag, status, 16);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        const uint32_t stage = sm.base_u32 + s * p.stage_bytes;
        const int i0 = beg + kc * kBK;
#pragma unroll 1
        for (int base = pt; base < tasks; base += 2 * np) {
          // two tasks per round: first both index lookups, then both row loads, then convert + store,
          // so that the two global-load latencies of a task overlap with the other task's
          float v[2][8];
          int r[2], c[2], tile[2], col[2];
          bool isb[2], live[2];
          int64_t row_off[2];
          float aux[2];          // input range (A) or gate scale (B)
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int task = base + b * np;
            live[b] = false;
            isb[b] = task >= a_tasks;
            r[b] = 0; c[b] = 0; tile[b] = 0; col[b] = 0; row_off[b] = 0; aux[b] = 1.f;
            if (task < tasks) {
              if (!isb[b]) { tile[b] = task >> 10; r[b] = (task >> 4) & 63; c[b] = task & 15; }
              else {
                int tt = task - a_tasks;
                tile[b] = tt >= b_tile_tasks ? 1 : 0;
                tt -= tile[b] * b_tile_tasks;
                if (b_shift >= 0) { r[b] = tt >> b_shift; c[b] = tt & (b_chunks - 1); }
                else { r[b] = tt / b_chunks; c[b] = tt - r[b] * b_chunks; }
              }
              const int i = i0 + r[b];
              if (i < end) {
                if (!isb[b]) {
                  col[b] = (mbk * p.MB + tile[b]) * kBM + c[b] * 8;
                  const int64_t xr = p.x_row[i];
                  if (xr < 0 || xr >= p.x_rows) report(status, AMOE_ERR_INDEX_RANGE, 30, i, static_cast<int>(xr));
                  else if (col[b] < p.K) {
                    live[b] = true;
                    row_off[b] = xr * p.x_stride;
                    if (p.ir) aux[b] = p.ir[p.ir_by_expert ? e : i];
                  }
                } else {
                  col[b] = (nbk * p.NB + tile[b]) * p.BN + c[b] * 8;
                  const int64_t gr = p.g_row[i];
                  const int64_t gsrc = p.g_div == 1 ? gr : gr / p.g_div;
                  if (gr < 0 || gsrc >= p.g_rows) report(status, AMOE_ERR_INDEX_RANGE, 31, i, static_cast<int>(gr));
                  else if (col[b] < p.N && c[b] * 8 < p.BN) {
                    live[b] = true;
                    row_off[b] = gsrc * p.g_stride;
                    if (p.g_scale) aux[b] = p.g_scale[gr];
                  }
                }
              }
            }
          }
#pragma unroll
          for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int x = 0; x < 8; ++x) v[b][x] = 0.f;
            if (live[b]) {
              const void* src = isb[b] ? p.g : p.x;
              const int lim = isb[b] ? p.N : p.K;
              if (IN == 0 && col[b] + 8 <= lim) load8_fast<true>(src, row_off[b], col[b], v[b]);
              else if (IN == 1 && col[b] + 8 <= lim) load8_fast<false>(src, row_off[b], col[b], v[b]);
              else load8(src, isb[b] ? p.g_dtype : p.x_dtype, row_off[b], col[b], lim,
                         IN != 2 || (isb[b] ? p.g_vec_ok : p.x_vec_ok) != 0, v[b]);
            }
          }
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            if (base + b * np < tasks) {
              if (live[b]) {
                if (!isb[b]) {
                  if (p.ir) {
#pragma unroll
                    for (int x = 0; x < 8; ++x) v[b][x] = clamp_ir(v[b][x], aux[b]);
                  }
                } else if (p.g_scale || p.f16) {
                  const float m = (p.g_scale ? aux[b] : 1.f) * g_mul;
#pragma unroll
                  for (int x = 0; x < 8; ++x) v[b][x] *= m;
                }
              }
              const uint32_t hi = stage + (isb[b] ? b_region + tile[b] * b_tile : tile[b] * a_tile);
              const uint32_t lo = hi + (isb[b] ? p.b_bytes : p.a_bytes);
              const uint32_t so = static_cast<uint32_t>((c[b] >> 3) * static_cast<int>(kMnBlock)) + sw128_offset(r[b], c[b] & 7);
              if (p.f16) store8_rt<true>(hi, lo, so, v[b], false);
              else store8<SPLIT>(hi, lo, so, v[b]);
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


// ---------------------------------------------------------------------------- dW from cached operands
// Both operands already exist in HBM as bf16 hi (+ lo) terms in padded tile-row order (written by the
// prologue of the forward kernel and by the prologue / epilogue of the input-gradient kernels): rows
// [128*t, 128*t+128) belong to tile t of the expert-sorted slot list, rows past an expert's last slot
// are zero.  The contraction runs over those rows, so the tiles come straight from TMA as MN-major
// operands and no thread touches the data before the tensor core does: six warps per CTA (TMA, MMA,
// four epilogue warps).

struct DwTmaParams {
  int E, K, N;
  int BN, m_tiles, n_tiles, stages;
  int MB, NB;
  int seg;              // padded rows per work segment (multiple of 64); 0: one segment per expert
  uint32_t tmem_cols, stage_bytes, a_bytes, b_bytes;
  const int32_t* offsets;
  float* dw;
  float* partials;
  int32_t* status;
  int f16;              // the caches hold fp16
  const float* g_absmax;  // device scalar max|g| behind the scale the g cache carries (dW is scaled back), or NULL
};

// Segment `idx` in padded row space: expert e owns ceil(count_e/128)*128 padded rows.
struct PadSegIter {
  const int32_t* off; int E, seg; int e; int64_t before; int64_t pad_base;
  __device__ PadSegIter(const int32_t* o, int E_, int seg_) : off(o), E(E_), seg(seg_), e(0), before(0), pad_base(0) {}
  __device__ bool get(int64_t idx, int& ex, int64_t& beg, int64_t& end) {
    while (e < E) {
      const int len = (off[e + 1] - off[e] + kBM - 1) / kBM * kBM;
      const int ns = seg > 0 ? (len + seg - 1) / seg : 1;
      if (idx < before + ns) {
        ex = e;
        beg = seg > 0 ? pad_base + (idx - before) * seg : pad_base;
        end = seg > 0 ? min(beg + seg, pad_base + len) : pad_base + len;
        return true;
      }
      before += ns;
      pad_base += len;
      ++e;
    }
    return false;
  }
};

constexpr int kDwTmaThreads = 6 * 32;

template <bool SPLIT>
__global__ void __launch_bounds__(kDwTmaThreads, 1)
dw_tc_tma_kernel(const __grid_constant__ CUtensorMap ta_hi, const __grid_constant__ CUtensorMap ta_lo,
                 const __grid_constant__ CUtensorMap tb_hi, const __grid_constant__ CUtensorMap tb_lo, DwTmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup_cta(sm, p.stages, p.tmem_cols, 1, 4);
  const uint32_t tmem_base = *sm.tmem_ptr;
  int32_t* status = p.status;
  const int mb_tiles = (p.m_tiles + p.MB - 1) / p.MB, nb_tiles = (p.n_tiles + p.NB - 1) / p.NB;
  const int tps = mb_tiles * nb_tiles;
  const int n_acc = p.MB * p.NB;
  const uint32_t a_tile = (SPLIT ? 2u : 1u) * p.a_bytes;
  const uint32_t b_tile = (SPLIT ? 2u : 1u) * p.b_bytes;
  const uint32_t b_region = static_cast<uint32_t>(p.MB) * a_tile;
  const int b_blocks = static_cast<int>(p.b_bytes / kMnBlock);
  float g_inv = 1.f;                    // the g cache carries the gradient scale of fp16 operands
  if (p.f16 && p.g_absmax != nullptr) grad_pow2_scale(__ldg(p.g_absmax), g_inv);
  const float out_mul = p.partials ? 1.f : g_inv;   // partial tiles keep it until dw_reduce_kernel

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&ta_hi); tma_prefetch_desc(&tb_hi);
      if (SPLIT) { tma_prefetch_desc(&ta_lo); tma_prefetch_desc(&tb_lo); }
      RingPos rp(p.stages);
      PadSegIter si(p.offsets, p.E, p.seg);
      const uint32_t tx_bytes = (SPLIT ? 2u : 1u) * (p.MB * 2u + p.NB * static_cast<uint32_t>(b_blocks)) * kMnBlock;
      bool alive = true;
      for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
        int e; int64_t beg, end;
        const int64_t seg_idx = w / tps;
        if (!si.get(seg_idx, e, beg, end)) break;
        const int sub = static_cast<int>(w - seg_idx * tps);
        const int nbk = sub % nb_tiles, mbk = sub / nb_tiles;
        const int chunks = static_cast<int>((end - beg) / kBK);
        for (int kc = 0; kc < chunks; ++kc, rp.next()) {
          const int s = rp.s;
          if (!mbar_wait(bar_empty(sm.bars, s), rp.ph ^ 1u, sm.abort_flag, status, 16, 32)) { alive = false; break; }
          const uint32_t stage = sm.base_u32 + s * p.stage_bytes;
          const uint32_t bar = bar_full_b(sm.bars, s);
          const int row = static_cast<int>(beg) + kc * kBK;
          mbar_arrive_expect_tx(bar, tx_bytes);
          for (int ma = 0; ma < p.MB; ++ma) {
            const int col = (mbk * p.MB + ma) * kBM;
            const uint32_t dst = stage + ma * a_tile;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              tma_load_3d(dst + blk * kMnBlock, &ta_hi, bar, 0, row, (col >> 6) + blk);
              if (SPLIT) tma_load_3d(dst + p.a_bytes + blk * kMnBlock, &ta_lo, bar, 0, row, (col >> 6) + blk);
            }
          }
          for (int nb = 0; nb < p.NB; ++nb) {
            const int col = (nbk * p.NB + nb) * p.BN;
            const uint32_t dst = stage + b_region + nb * b_tile;
            for (int blk = 0; blk < b_blocks; ++blk) {
              tma_load_3d(dst + blk * kMnBlock, &tb_hi, bar, 0, row, (col >> 6) + blk);
              if (SPLIT) tma_load_3d(dst + p.b_bytes + blk * kMnBlock, &tb_lo, bar, 0, row, (col >> 6) + blk);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = p.f16 ? (make_idesc_f16(kBM, p.BN) | (1u << 15) | (1u << 16)) : make_idesc_bf16_mn(kBM, p.BN);
      RingPos rp(p.stages);
      PadSegIter si(p.offsets, p.E, p.seg);
      uint32_t acc_it = 0;
      bool alive = true;
      for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
        int e; int64_t beg, end;
        if (!si.get(w / tps, e, beg, end)) break;
        const int chunks = static_cast<int>((end - beg) / kBK);
        if (chunks == 0) continue;
        const int buf = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(bar_tempty(sm.bars, buf), aph ^ 1u, sm.abort_flag, status, 12)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_base = tmem_base + static_cast<uint32_t>(buf * n_acc * p.BN);
        for (int kc = 0; kc < chunks; ++kc, rp.next()) {
          const int s = rp.s;
          if (!mbar_wait(bar_full_b(sm.bars, s), rp.ph, sm.abort_flag, status, 13)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = sm.base_u32 + s * p.stage_bytes;
          for (int acc = 0; acc < n_acc; ++acc) {
            const int ma = acc / p.NB, nb = acc - ma * p.NB;
            const uint32_t at = sa + ma * a_tile, bt = sa + b_region + nb * b_tile;
            const uint64_t da_hi = make_smem_desc_mn_sw128(at, kMnBlock);
            const uint64_t da_lo = make_smem_desc_mn_sw128(at + p.a_bytes, kMnBlock);
            const uint64_t db_hi = make_smem_desc_mn_sw128(bt, kMnBlock);
            const uint64_t db_lo = make_smem_desc_mn_sw128(bt + p.b_bytes, kMnBlock);
            const uint32_t d_tmem = d_base + static_cast<uint32_t>(acc * p.BN);
#pragma unroll
            for (int k16 = 0; k16 < kBK / 16; ++k16) {
              const uint64_t adv = static_cast<uint64_t>(k16 * (16 * 128 / 16));
              umma_bf16(d_tmem, da_hi + adv, db_hi + adv, idesc, (kc | k16) != 0 ? 1u : 0u);
              if (SPLIT) {
                umma_bf16(d_tmem, da_hi + adv, db_lo + adv, idesc, 1u);
                umma_bf16(d_tmem, da_lo + adv, db_hi + adv, idesc, 1u);
              }
            }
          }
          umma_commit(bar_empty(sm.bars, s));
        }
        if (alive) umma_commit(bar_tfull(sm.bars, buf));
        ++acc_it;
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    PadSegIter si(p.offsets, p.E, p.seg);
    uint32_t acc_it = 0;
    bool alive = true;
    for (int64_t w = blockIdx.x; alive; w += gridDim.x) {
      int e; int64_t beg, end;
      const int64_t seg_idx = w / tps;
      if (!si.get(seg_idx, e, beg, end)) break;
      const int sub = static_cast<int>(w - seg_idx * tps);
      const int nbk = sub % nb_tiles, mbk = sub / nb_tiles;
      const int chunks = static_cast<int>((end - beg) / kBK);
      float* out_base = p.partials ? p.partials + seg_idx * p.K * p.N : p.dw + static_cast<int64_t>(e) * p.K * p.N;
      if (chunks == 0) {   // only without segment splitting: an expert nobody was routed to
        for (int acc = 0; acc < n_acc; ++acc) {
          const int ma = acc / p.NB, nb = acc - ma * p.NB;
          const int m = (mbk * p.MB + ma) * kBM + r, n0 = (nbk * p.NB + nb) * p.BN;
          if (m < p.K)
            for (int n = n0; n < min(n0 + p.BN, p.N); ++n) out_base[static_cast<int64_t>(m) * p.N + n] = 0.f;
        }
        continue;
      }
      const int buf = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      bool ok = mbar_wait(bar_tfull(sm.bars, buf), aph, sm.abort_flag, status, 15, 64);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      for (int acc = 0; acc < n_acc; ++acc) {
        const int ma = acc / p.NB, nb = acc - ma * p.NB;
        const int m = (mbk * p.MB + ma) * kBM + r, n0 = (nbk * p.NB + nb) * p.BN;
        float* dst = out_base + static_cast<int64_t>(m) * p.N;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               static_cast<uint32_t>((buf * n_acc + acc) * p.BN);
#pragma unroll 1
        for (int c0 = 0; c0 < p.BN; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 16; ++x) v[x] *= out_mul;
          const int n = n0 + c0;
          if (m < p.K && n < p.N) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(sm.bars, buf));
      ++acc_it;
    }
  }
  teardown_cta(sm, tmem_base, p.tmem_cols);
}

// dW[e] = sum over the expert's segments, in segment order (fixed order: bit-reproducible).  `pad`: the
// segments were cut in padded row space (every expert's count rounded up to a multiple of `pad`).
__global__ void dw_reduce_kernel(const float* __restrict__ partials, const int32_t* __restrict__ offsets, int E, int seg,
                                 int64_t kn, float* __restrict__ dw, int pad, const float* __restrict__ g_absmax) {
  __shared__ int s_first, s_count;
  const int e = blockIdx.y;
  if (threadIdx.x == 0) {
    int first = 0;
    for (int x = 0; x < e; ++x) first += ((offsets[x + 1] - offsets[x] + pad - 1) / pad * pad + seg - 1) / seg;
    s_first = first;
    s_count = ((offsets[e + 1] - offsets[e] + pad - 1) / pad * pad + seg - 1) / seg;
  }
  __syncthreads();
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= kn) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sgm = 0; sgm < s_count; ++sgm) {
    const float4 v = *reinterpret_cast<const float4*>(partials + (static_cast<int64_t>(s_first) + sgm) * kn + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (g_absmax != nullptr) {      // fp16 operands: the partial tiles still carry the gradient scale
    float inv;
    grad_pow2_scale(__ldg(g_absmax), inv);
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  *reinterpret_cast<float4*>(dw + static_cast<int64_t>(e) * kn + i) = acc;
}

// Slots per segment for the split, or 0 when the work is too small to be worth splitting.
// A work item is (segment, pair of output tiles).  The segment length is chosen so that the items of a balanced
// routing fill the SMs about once - every further wave adds a set of partial tiles to write and sum, and short items
// (a few 64-slot stages) do not amortise the latency of their first loads - and so that an expert's expected share
// divides into equal segments.  Experts with more rows simply get more segments.
int dw_segment_slots(int64_t P, int E, int K, int N) {
  if (P <= 4096 || (static_cast<int64_t>(K) * N) % 4 != 0) return 0;
  const int n_pad = round_up(N, 16);
  const int n_tiles = (n_pad + 127) / 128;
  const int m_tiles = (K + kBM - 1) / kBM;
  int MB = 1, NB = 1;
  if (m_tiles >= 2 && m_tiles >= n_tiles) MB = 2;
  else if (n_tiles >= 2) NB = 2;
  const int64_t pairs = static_cast<int64_t>((m_tiles + MB - 1) / MB) * ((n_tiles + NB - 1) / NB);
  const int64_t per_expert = P / (E > 0 ? E : 1) + kBM;          // expected padded rows of an expert
  int64_t target = (P + static_cast<int64_t>(kBM) * E) * pairs / 148;   // rows per item for one wave
  if (target < 512) target = 512;
  int64_t n = (per_expert + target / 2) / target;                 // segments per (balanced) expert, rounded
  if (n < 1) n = 1;
  int64_t seg = (per_expert + n - 1) / n;
  seg = (seg + 63) / 64 * 64;
  if (seg < 256) seg = 256;
  if (seg > 4096) seg = 4096;
  return static_cast<int>(seg);
}

uint32_t pow2_cols(int need) {
  uint32_t c = 32;
  while (static_cast<int>(c) < need) c <<= 1;
  return c;
}

constexpr uint32_t kSmemBudget = 196 * 1024;  // ring budget; barriers and alignment slack come on top
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
  const bool f16 = a->precision == AMOE_PREC_F16X1;
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
  p.ir = is_dx ? nullptr : a->ir;
  p.a_absmax = is_dx ? nullptr : a->a_absmax;
  p.inp_res = is_dx ? -1.f : a->inp_res;
  const int esz = a->a_dtype == AMOE_F32 ? 4 : 2;
  p.vec_ok = aligned16(a->a) && ((a->a_stride * esz) % 16 == 0);
  p.epi = epi_in;
  p.g_absmax = (f16 && is_dx) ? a->a_absmax_dev : nullptr;
  const bool dac = !is_dx;
  const bool quant = dac && p.inp_res > 0.f;
  // Integer DAC codes up to 256 in magnitude are exact in bf16 (up to 2048 in fp16); anything else needs the hi+lo
  // pair when split precision is asked for.  bf16 inputs that are not quantised are exact as they are.
  bool a_split = a->precision == AMOE_PREC_SPLIT;
  if (quant && p.inp_res >= 1.0f / 256.0f) a_split = false;
  if (!quant && a->a_dtype == AMOE_BF16 && !(dac && (p.ir || p.a_absmax))) a_split = false;
  const bool b_split = a->precision == AMOE_PREC_SPLIT && a->w_lo != nullptr;
  p.a_split = a_split; p.b_split = b_split;
  p.epi.acc_mul = quant ? p.inp_res : 1.f;
  p.cache_hi = reinterpret_cast<__nv_bfloat16*>(a->a_cache_hi);
  p.cache_lo = f16 ? nullptr : reinterpret_cast<__nv_bfloat16*>(a->a_cache_lo);
  p.cache_stride = a->cache_rows; p.cache_scale = a->a_cache_scale;
  p.a_tma = a->a_tile_hi != nullptr;
  if (p.a_tma) {
    AMOE_REQUIRE(p.Kc % kBK == 0 && aligned16(a->a_tile_hi) && aligned16(a->a_tile_lo) && !p.cache_hi, AMOE_ERR_BAD_SHAPE);
    AMOE_REQUIRE(a->cache_rows >= (a->P / kBM + a->E) * kBM, AMOE_ERR_BAD_SHAPE);
    a_split = !f16 && a->a_tile_lo != nullptr;
    p.a_split = a_split;
  }
  AMOE_REQUIRE(!(p.cache_hi || p.epi.out_cache_hi || p.epi.next_codes) || a->cache_rows >= (a->P / kBM + a->E) * kBM, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(!p.cache_hi || (p.Kc % 8 == 0 && aligned16(p.cache_hi) && aligned16(p.cache_lo)), AMOE_ERR_BAD_SHAPE);
  if (f16) p.epi.out_cache_lo = nullptr;

  p.a_bytes = a_split ? 2 * kATile : kATile;
  // exchange blocks per epilogue warp: one, or two where the clip-reference rows are prefetched
  const bool xpre = is_dx && a->x_ref != nullptr;
  const uint32_t tr_unit = kTrBytesPerWarp * (xpre ? 2u : 1u);
  // two ring stages must fit beside the epilogue warps' exchange blocks: wide weight tiles in two terms are cut into
  // narrower n-tiles where they do not
  for (;;) {
    p.b_bytes = static_cast<uint32_t>(p.BN) * 128u;
    p.stage_bytes = p.a_bytes + p.b_bytes * (b_split ? 2u : 1u);
    p.stage_bytes = (p.stage_bytes + 1023u) & ~1023u;
    if ((kSmemBudget - 4u * tr_unit) / p.stage_bytes >= 2 || p.BN <= 64) break;     // (four epilogue warps at the least)
    p.n_tiles *= 2;
    p.BN = round_up((n_pad + p.n_tiles - 1) / p.n_tiles, 16);
  }
  p.item_mode = p.a_tma && !is_dx && p.n_tiles > 1;
  p.tmem_cols = pow2_cols(2 * p.BN);
  p.prod_groups = 1;
  {
    // Split the worker warps between epilogue and prologue by estimated instruction counts.
    const double per_prod = (quant ? 8.0 : (dac && (p.ir || p.a_absmax) ? 10.0 : 2.0)) + (a_split ? 5.0 : 2.0) +
                            (p.cache_hi ? (f16 ? 2.0 : 5.0) : 0.0);
    double per_epi = 8.0;
    if (!is_dx) per_epi += (a->noise_std > 0.f ? 26.0 : 0.0) + (a->noise ? 2.0 : 0.0) + (p.epi.adc.on ? 9.0 : 0.0) +
                           (a->out_codes ? 3.0 : 0.0) + (p.epi.next_codes ? 14.0 : 0.0) + (p.epi.out_cache_hi ? 10.0 : 0.0);
    else per_epi += a->x_ref ? 12.0 : 0.0;
    const double work_p = static_cast<double>(p.n_tiles) * p.k_chunks * kBK * per_prod;
    const double work_e = static_cast<double>(p.n_tiles) * p.BN * per_epi;
    double best = 1e300;
    auto fits = [&](int ne) { return (kSmemBudget - static_cast<uint32_t>(ne) * tr_unit) / p.stage_bytes >= 2; };
    p.n_epi = 4; p.n_prod = kWorkerWarps - 4;
    for (int ne = 4; ne <= kWorkerWarps - 2 && ne <= 24; ne += 4) {
      if (!fits(ne)) continue;
      const double t = fmax(work_p / (kWorkerWarps - ne), work_e / ne);
      if (t < best) { best = t; p.n_epi = ne; p.n_prod = kWorkerWarps - ne; }
    }
    if (p.a_tma) {
      // no prologue: the epilogue groups that share the tile's chunks most evenly (fewest warps on a tie)
      const int chunks = p.BN / 16;
      int best_per = 1 << 30;
      for (int ne = 4; ne <= kWorkerWarps; ne += 4) {
        if (!fits(ne)) continue;
        const int per = (chunks + ne / 4 - 1) / (ne / 4);
        if (per < best_per) { best_per = per; p.n_epi = ne; }
      }
      p.n_prod = 0;
    }
  }
  // the ring takes what the epilogue warps' exchange blocks leave of the budget
  const uint32_t tr_bytes = static_cast<uint32_t>(p.n_epi) * tr_unit;
  p.stages = static_cast<int>((kSmemBudget - tr_bytes) / p.stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  AMOE_REQUIRE(p.stages >= 2, AMOE_ERR_UNSUPPORTED);
  // prologue warps: two groups on alternate stages (both groups have the same number of warps, so every stage's
  // barrier expects the same number of arrivals whichever group fills it); needs enough stages per tile to alternate on
  if (!p.a_tma && p.stages >= 3 && p.k_chunks * p.n_tiles >= 4 && p.n_prod >= 8 && p.n_prod % 2 == 0)
    p.prod_groups = 2;
  // per-warp staging of the column scales: chunks per warp x 16 floats, two arrays
  {
    const int groups = p.n_epi / 4;
    p.cs_per_warp = ((p.BN / 16 + groups - 1) / groups) * 16;
    p.cs_off = static_cast<uint32_t>(p.stages) * p.stage_bytes + 8u * kNumBars + 64u;
  }
  const uint32_t cs_bytes = static_cast<uint32_t>(p.n_epi) * 2u * p.cs_per_warp * sizeof(float);

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
  CUtensorMap ma_hi = m_hi, ma_lo = m_hi;
  if (p.a_tma) {
    s = encode_tmap_bf16_3d(&ma_hi, a->a_tile_hi, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>(p.Kc / kBK), 64, kBM);
    if (s != AMOE_OK) return s;
    ma_lo = ma_hi;
    if (a_split) {
      s = encode_tmap_bf16_3d(&ma_lo, a->a_tile_lo, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>(p.Kc / kBK), 64, kBM);
      if (s != AMOE_OK) return s;
    }
  }
  p.tr_off = (p.cs_off + cs_bytes + 15u) & ~15u;
  const uint32_t smem = p.tr_off + tr_bytes + kSmemExtra;
  const int64_t max_tiles = ((a->P + kBM - 1) / kBM + a->E) * (p.item_mode ? p.n_tiles : 1);
  const int grid = static_cast<int>(max_tiles < sm_count() ? max_tiles : sm_count());
  const bool f32 = a->a_dtype == AMOE_F32;
  // epilogue family: the fast routines need 16-byte alignment everywhere and no materialised noise
  int epi = kEpiGeneric;
  if (p.epi.vec4 && !is_dx && a->noise == nullptr) epi = kEpiFwd;
  if (p.epi.vec4 && is_dx && (a->x_ref == nullptr || a->x_ref_dtype == AMOE_F32 || a->x_ref_stride % 8 == 0)) epi = kEpiDx;
  AMOE_REQUIRE(!(p.epi.out_cache_hi || p.epi.next_codes) || epi == (is_dx ? kEpiDx : kEpiFwd), AMOE_ERR_UNSUPPORTED);
  AMOE_REQUIRE(a->out != nullptr || epi != kEpiGeneric, AMOE_ERR_UNSUPPORTED);
  const int dacm = is_dx ? kDacNone : (quant ? kDacQuant : kDacNorm);
#define AMOE_LAUNCH_TC(DAC, F32, EPI, F16)                                                                                  \
  do {                                                                                                                      \
    AMOE_CUDA(cudaFuncSetAttribute(cvmm_tc_kernel<DAC, F32, EPI, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    cvmm_tc_kernel<DAC, F32, EPI, F16><<<grid, kFwdThreads, smem, stream>>>(m_hi, m_lo, ma_hi, ma_lo, p);                   \
  } while (0)
#define AMOE_LAUNCH_TC_DT(DAC, EPI)                                                                 \
  do {                                                                                              \
    if (f16) { if (f32) AMOE_LAUNCH_TC(DAC, true, EPI, true); else AMOE_LAUNCH_TC(DAC, false, EPI, true); }   \
    else { if (f32) AMOE_LAUNCH_TC(DAC, true, EPI, false); else AMOE_LAUNCH_TC(DAC, false, EPI, false); }     \
  } while (0)
  if (is_dx) {
    if (epi == kEpiDx) AMOE_LAUNCH_TC_DT(kDacNone, kEpiDx); else AMOE_LAUNCH_TC_DT(kDacNone, kEpiGeneric);
  } else if (dacm == kDacQuant) {
    if (epi == kEpiFwd) AMOE_LAUNCH_TC_DT(kDacQuant, kEpiFwd); else AMOE_LAUNCH_TC_DT(kDacQuant, kEpiGeneric);
  } else {
    if (epi == kEpiFwd) AMOE_LAUNCH_TC_DT(kDacNorm, kEpiFwd); else AMOE_LAUNCH_TC_DT(kDacNorm, kEpiGeneric);
  }
#undef AMOE_LAUNCH_TC_DT
#undef AMOE_LAUNCH_TC
  AMOE_LAUNCH_CHECK("cvmm_tc");
  return AMOE_OK;
}

// A wait that nothing ends: one warp waits, with the kernels' own bounded wait, on an mbarrier that no one arrives
// at; the wait gives up after `limit_cycles`, records AMOE_ERR_WAIT_LIMIT in the status word and the kernel returns
// normally.  This is how the give-up path of the pipelines is exercised without stalling a GPU.
__global__ void bounded_wait_selftest_kernel(int32_t* status, long long limit_cycles) {
  using namespace tc;
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < 32) ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, status, 99, 32, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && ok) report(status, AMOE_ERR_UNSUPPORTED, 99, 0, 0);   // the wait must not have succeeded
}

}  // namespace amoe

extern "C" int amoe_selftest_bounded_wait(int32_t* dev_status, long long limit_cycles, amoe_stream_t stream_) {
  using namespace amoe;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(dev_status != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(limit_cycles > 0 && limit_cycles <= 4000000000LL, AMOE_ERR_BAD_SHAPE);
  int s = amoe_check_device();
  if (s != AMOE_OK) return s;
  bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(dev_status, limit_cycles);
  AMOE_LAUNCH_CHECK("bounded_wait_selftest");
  return AMOE_OK;
}

namespace amoe {

size_t dw_tc_workspace_bytes(int64_t P, int64_t expected, int E, int K, int N) {
  const int seg = dw_segment_slots(expected > 0 && expected < P ? expected : P, E, K, N);
  if (seg == 0) return 0;
  // segments are cut per expert, in padded row space when the operands come from the caches
  return static_cast<size_t>((P + static_cast<int64_t>(kBM) * E + seg - 1) / seg + E) * K * N * sizeof(float);
}

static int launch_dw_tma(const amoe_dw_args* a, cudaStream_t stream) {
  DwTmaParams p{};
  p.E = a->E; p.K = a->K; p.N = a->N;
  // output tiles start on 64-column blocks of the cache layout
  p.BN = a->N > 64 ? 128 : 64;
  p.n_tiles = (a->N + p.BN - 1) / p.BN;
  p.m_tiles = (a->K + kBM - 1) / kBM;
  p.offsets = a->expert_offsets;
  p.dw = a->dw; p.status = a->dev_status;
  p.f16 = a->precision == AMOE_PREC_F16X1; p.g_absmax = a->g_absmax_dev;
  const int64_t tune = a->expected_rows > 0 && a->expected_rows < a->P ? a->expected_rows : a->P;
  p.seg = dw_segment_slots(tune, a->E, a->K, a->N);
  const size_t need = dw_tc_workspace_bytes(a->P, tune, a->E, a->K, a->N);
  if (p.seg > 0 && (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace) || !aligned16(a->dw)))
    p.seg = 0;
  p.partials = p.seg > 0 ? reinterpret_cast<float*>(a->workspace) : nullptr;
  const bool split = !p.f16 && a->x_lo != nullptr && a->g_lo != nullptr;
  AMOE_REQUIRE(split || p.f16 || (a->x_lo == nullptr && a->g_lo == nullptr), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(aligned16(a->x_hi) && aligned16(a->x_lo) && aligned16(a->g_hi) && aligned16(a->g_lo), AMOE_ERR_BAD_SHAPE);
  p.a_bytes = 2 * kMnBlock;
  p.b_bytes = static_cast<uint32_t>((p.BN + 63) / 64) * kMnBlock;
  p.MB = 1; p.NB = 1;
  if (p.m_tiles >= 2 && p.m_tiles >= p.n_tiles) p.MB = 2;
  else if (p.n_tiles >= 2) p.NB = 2;
  p.stage_bytes = (split ? 2u : 1u) * (p.MB * p.a_bytes + p.NB * p.b_bytes);
  p.stages = static_cast<int>(kSmemBudget / p.stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  AMOE_REQUIRE(p.stages >= 2, AMOE_ERR_UNSUPPORTED);
  p.tmem_cols = pow2_cols(2 * p.MB * p.NB * p.BN);
  const uint32_t smem = p.stages * p.stage_bytes + kSmemExtra;
  const int64_t pad_rows = a->P + static_cast<int64_t>(kBM) * a->E;
  const int64_t segs = p.seg > 0 ? (pad_rows + p.seg - 1) / p.seg + a->E : a->E;
  const int64_t items = segs * ((p.m_tiles + p.MB - 1) / p.MB) * ((p.n_tiles + p.NB - 1) / p.NB);
  const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
  int s = encode_tmap_bf16_3d(&ta_hi, a->x_hi, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>((a->K + 63) / 64), 64, kBK);
  if (s != AMOE_OK) return s;
  s = encode_tmap_bf16_3d(&tb_hi, a->g_hi, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>((a->N + 63) / 64), 64, kBK);
  if (s != AMOE_OK) return s;
  ta_lo = ta_hi; tb_lo = tb_hi;
  if (split) {
    s = encode_tmap_bf16_3d(&ta_lo, a->x_lo, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>((a->K + 63) / 64), 64, kBK);
    if (s != AMOE_OK) return s;
    s = encode_tmap_bf16_3d(&tb_lo, a->g_lo, 64, static_cast<uint64_t>(a->cache_rows), static_cast<uint64_t>((a->N + 63) / 64), 64, kBK);
    if (s != AMOE_OK) return s;
  }
  if (split) {
    AMOE_CUDA(cudaFuncSetAttribute(dw_tc_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dw_tc_tma_kernel<true><<<grid, kDwTmaThreads, smem, stream>>>(ta_hi, ta_lo, tb_hi, tb_lo, p);
  } else {
    AMOE_CUDA(cudaFuncSetAttribute(dw_tc_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dw_tc_tma_kernel<false><<<grid, kDwTmaThreads, smem, stream>>>(ta_hi, ta_lo, tb_hi, tb_lo, p);
  }
  AMOE_LAUNCH_CHECK("dw_tc_tma");
  if (p.seg > 0) {
    const int64_t kn = static_cast<int64_t>(a->K) * a->N;
    dim3 rg(static_cast<unsigned>((kn / 4 + 255) / 256), a->E);
    dw_reduce_kernel<<<rg, 256, 0, stream>>>(p.partials, p.offsets, a->E, p.seg, kn, a->dw, kBM, p.f16 ? p.g_absmax : nullptr);
    AMOE_LAUNCH_CHECK("dw_reduce");
  }
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
  p.ir = a->ir; p.ir_by_expert = a->ir_by_expert;
  p.g = a->g; p.g_dtype = a->g_dtype; p.g_stride = a->g_stride; p.g_rows = a->g_rows; p.g_row = a->g_row;
  p.g_div = a->g_div < 1 ? 1 : a->g_div; p.g_scale = a->g_scale;
  p.x_vec_ok = aligned16(a->x) && ((a->x_stride * (a->x_dtype == AMOE_F32 ? 4 : 2)) % 16 == 0);
  p.g_vec_ok = aligned16(a->g) && ((a->g_stride * (a->g_dtype == AMOE_F32 ? 4 : 2)) % 16 == 0);
  p.dw = a->dw; p.status = a->dev_status;
  p.f16 = a->precision == AMOE_PREC_F16X1; p.g_absmax = a->g_absmax_dev;
  if (a->x_hi != nullptr) return launch_dw_tma(a, stream);
  // Large problems: cut every expert's slot range into segments so that the work items outnumber the
  // SMs and a popular expert does not become one long item; the partial tiles go to the workspace and
  // are summed in segment order afterwards.
  const int64_t tune = a->expected_rows > 0 && a->expected_rows < a->P ? a->expected_rows : a->P;
  p.seg = dw_segment_slots(tune, a->E, a->K, a->N);
  const size_t need = dw_tc_workspace_bytes(a->P, tune, a->E, a->K, a->N);
  if (p.seg > 0 && (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace) || !aligned16(a->dw)))
    p.seg = 0;   // no (usable) workspace: one owner per expert tile
  p.partials = p.seg > 0 ? reinterpret_cast<float*>(a->workspace) : nullptr;
  // bf16 inputs are exact in one term; fp32 inputs are split unless the caller asked for the fast mode
  const bool split = a->precision == AMOE_PREC_SPLIT && !(a->x_dtype == AMOE_BF16 && a->g_dtype == AMOE_BF16 && !a->g_scale);
  p.a_bytes = 2 * kMnBlock;                                             // 128 columns = 2 blocks
  p.b_bytes = static_cast<uint32_t>((p.BN + 63) / 64) * kMnBlock;
  // two output tiles per work item along the longer tile dimension, when there are at least two
  p.MB = 1; p.NB = 1;
  if (p.m_tiles >= 2 && p.m_tiles >= p.n_tiles) p.MB = 2;
  else if (p.n_tiles >= 2) p.NB = 2;
  p.stage_bytes = (split ? 2u : 1u) * (p.MB * p.a_bytes + p.NB * p.b_bytes);
  p.stages = static_cast<int>(kSmemBudget / p.stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  AMOE_REQUIRE(p.stages >= 2, AMOE_ERR_UNSUPPORTED);
  p.tmem_cols = pow2_cols(2 * p.MB * p.NB * p.BN);
  const uint32_t smem = p.stages * p.stage_bytes + kSmemExtra;
  const int64_t segs = p.seg > 0 ? (a->P + p.seg - 1) / p.seg + a->E : a->E;
  const int64_t items = segs * ((p.m_tiles + p.MB - 1) / p.MB) * ((p.n_tiles + p.NB - 1) / p.NB);
  const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
  int in_class = 2;
  if (p.x_vec_ok && p.g_vec_ok && a->x_dtype == AMOE_F32 && a->g_dtype == AMOE_F32) in_class = 0;
  if (p.x_vec_ok && p.g_vec_ok && a->x_dtype == AMOE_BF16 && a->g_dtype == AMOE_BF16) in_class = 1;
#define AMOE_LAUNCH_DW(SP, IN)                                                                                       \
  do {                                                                                                               \
    AMOE_CUDA(cudaFuncSetAttribute(dw_tc_mn_kernel<SP, IN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));    \
    dw_tc_mn_kernel<SP, IN><<<grid, kDwThreads, smem, stream>>>(p);                                                  \
  } while (0)
  if (split) {
    if (in_class == 0) AMOE_LAUNCH_DW(true, 0); else if (in_class == 1) AMOE_LAUNCH_DW(true, 1); else AMOE_LAUNCH_DW(true, 2);
  } else {
    if (in_class == 0) AMOE_LAUNCH_DW(false, 0); else if (in_class == 1) AMOE_LAUNCH_DW(false, 1); else AMOE_LAUNCH_DW(false, 2);
  }
#undef AMOE_LAUNCH_DW
  AMOE_LAUNCH_CHECK("dw_tc");
  if (p.seg > 0) {
    const int64_t kn = static_cast<int64_t>(a->K) * a->N;
    dim3 rg(static_cast<unsigned>((kn / 4 + 255) / 256), a->E);
    dw_reduce_kernel<<<rg, 256, 0, stream>>>(p.partials, p.offsets, a->E, p.seg, kn, a->dw, 1, p.f16 ? p.g_absmax : nullptr);
    AMOE_LAUNCH_CHECK("dw_reduce");
  }
  return AMOE_OK;
}

}  // namespace amoe
