// The router around the CVMM path: gate logits (a skinny matrix product), the weight gradient of the
// router from the expert-sorted slot list, and the sum over k of the input gradient with the router's own
// input-gradient term folded in.  CUDA-core fp32 throughout: T x D x E is far too thin for the tensor core
// to matter, the kernels are bound by reading x once.
#include "common.cuh"

namespace amoe {
namespace {

// ------------------------------------------------------------------------------------ logits
// logits[t,e] = sum_d x[t,d] * w[e,d] (+ bias[e]).  Block: 128 threads, kTok tokens x up to 64 experts; a thread
// owns 2 tokens x 4 experts.  The contraction runs in chunks of 32 columns through shared memory, the next
// chunk's global loads are issued before the current chunk is multiplied.
constexpr int kRk = 32;            // contraction chunk
constexpr int kRPad = kRk + 4;     // row pitch in shared memory (floats): 16-byte aligned, conflict-free

template <typename T>
__device__ __forceinline__ float4 ldg4(const T* p, bool vec, int valid) {
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  if (valid <= 0) return o;
  if (vec && valid >= 4) {
    if constexpr (sizeof(T) == 4) {
      o = __ldg(reinterpret_cast<const float4*>(p));
    } else {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
      o = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                      __uint_as_float(u.y & 0xffff0000u));
    }
  } else {
    o.x = to_f32<T>(p[0]);
    if (valid > 1) o.y = to_f32<T>(p[1]);
    if (valid > 2) o.z = to_f32<T>(p[2]);
    if (valid > 3) o.w = to_f32<T>(p[3]);
  }
  return o;
}

// EQ = expert quads per block (1, 2, 4, 8 or 16): the block covers 4*EQ experts and 2 * (128 / EQ) tokens.
template <typename TX, typename TW, int EQ>
__global__ void __launch_bounds__(128) router_logits_kernel(const TX* __restrict__ x, int64_t x_stride, int64_t T, int D,
                                                            const TW* __restrict__ w, int E,
                                                            const float* __restrict__ bias, int round_bf16,
                                                            float* __restrict__ logits, int vec) {
  constexpr int kTq = 128 / EQ;        // token pairs per block
  constexpr int kTok = 2 * kTq;
  constexpr int kExp = 4 * EQ;
  __shared__ __align__(16) float xs[kTok][kRPad];
  __shared__ __align__(16) float ws[kExp][kRPad];
  const int tid = threadIdx.x;
  const int eq = tid % EQ, tq = tid / EQ;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * kTok;
  const int e0 = blockIdx.y * kExp;
  // load roles: 8 threads cover the 32 columns of a row
  const int lr = tid >> 3, lc = (tid & 7) * 4;
  constexpr int kXPasses = kTok / 16, kWPasses = (kExp + 15) / 16;
  float4 xr[kXPasses], wr[kWPasses];
  auto load_chunk = [&](int d0) {
#pragma unroll
    for (int ps = 0; ps < kXPasses; ++ps) {
      const int64_t t = t0 + lr + 16 * ps;
      xr[ps] = t < T ? ldg4<TX>(x + t * x_stride + d0 + lc, vec != 0, D - d0 - lc) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int ps = 0; ps < kWPasses; ++ps) {
      const int e = e0 + lr + 16 * ps;
      wr[ps] = (e < E && lr + 16 * ps < kExp) ? ldg4<TW>(w + static_cast<int64_t>(e) * D + d0 + lc, vec != 0, D - d0 - lc)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  load_chunk(0);
  for (int d0 = 0; d0 < D; d0 += kRk) {
    __syncthreads();     // the previous chunk has been consumed
#pragma unroll
    for (int ps = 0; ps < kXPasses; ++ps) *reinterpret_cast<float4*>(&xs[lr + 16 * ps][lc]) = xr[ps];
#pragma unroll
    for (int ps = 0; ps < kWPasses; ++ps)
      if (lr + 16 * ps < kExp) *reinterpret_cast<float4*>(&ws[lr + 16 * ps][lc]) = wr[ps];
    __syncthreads();
    if (d0 + kRk < D) load_chunk(d0 + kRk);
#pragma unroll
    for (int kq = 0; kq < kRk / 4; ++kq) {
      float4 a[2], b[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = *reinterpret_cast<const float4*>(&xs[2 * tq + i][4 * kq]);
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(&ws[4 * eq + j][4 * kq]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t t = t0 + 2 * tq + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + 4 * eq + j;
      if (e < E) {
        float v = acc[i][j];
        if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        if (bias) v += bias[e];
        if (round_bf16 && bias) v = __bfloat162float(__float2bfloat16_rn(v));
        logits[t * E + e] = v;
      }
    }
  }
}

// Routers whose weight fits in shared memory (the usual case: tens of experts): the weight is staged once per
// block as fp32, a warp takes two tokens at a time, every lane multiplies its four columns of each 128-column step
// against 16 experts from shared memory, and the 2 x 16 partial sums meet in one 31-shuffle butterfly that leaves
// value (token, expert) = lane in lane `lane`.  Reads x exactly once with 16-byte loads.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) router_logits_smem_kernel(const TX* __restrict__ x, int64_t x_stride, int64_t T, int D,
                                                                 const TW* __restrict__ w, int E,
                                                                 const float* __restrict__ bias, int round_bf16,
                                                                 float* __restrict__ logits, int k, int apply_sigmoid,
                                                                 int32_t* __restrict__ raw_sel, float* __restrict__ gate) {
  extern __shared__ __align__(16) float s_w[];        // [ceil16(E)][D], rows past E are zero
  const int Ep = (E + 15) / 16 * 16;
  for (int i = threadIdx.x * 4; i < Ep * D; i += 1024) {
    const int e = i / D, d = i - e * D;
    const float4 v = e < E ? ldg4<TW>(w + static_cast<int64_t>(e) * D + d, true, 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(s_w + i) = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
  const int64_t pairs = (T + 1) / 2;
  for (int64_t pr = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); pr < pairs; pr += warps) {
    const int64_t t0 = 2 * pr;
    const bool two = t0 + 1 < T;
    const TX* x0 = x + t0 * x_stride;
    const TX* x1 = x + (two ? t0 + 1 : t0) * x_stride;
    float picks[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // this lane's gate values, expert 16*i + (lane & 15)
    for (int e0 = 0; e0 < Ep; e0 += 16) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll 2
      for (int d = lane * 4; d < D; d += 128) {
        const float4 a = ldg4<TX>(x0 + d, true, 4), b = ldg4<TX>(x1 + d, true, 4);
        const float* wp = s_w + static_cast<size_t>(e0) * D + d;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float4 ww = *reinterpret_cast<const float4*>(wp + static_cast<size_t>(e) * D);
          v[e] = fmaf(a.x, ww.x, v[e]); v[e] = fmaf(a.y, ww.y, v[e]); v[e] = fmaf(a.z, ww.z, v[e]); v[e] = fmaf(a.w, ww.w, v[e]);
          v[16 + e] = fmaf(b.x, ww.x, v[16 + e]); v[16 + e] = fmaf(b.y, ww.y, v[16 + e]);
          v[16 + e] = fmaf(b.z, ww.z, v[16 + e]); v[16 + e] = fmaf(b.w, ww.w, v[16 + e]);
        }
      }
      // butterfly: after the level with offset o the lanes whose bit o is set keep the upper half of the values
#pragma unroll
      for (int o = 16, n = 32; o >= 1; o >>= 1, n >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          const float lo_v = v[i], hi_v = v[i + n / 2];
          const float recv = __shfl_xor_sync(0xffffffffu, up ? lo_v : hi_v, o);
          v[i] = (up ? hi_v : lo_v) + recv;
        }
      }
      const int64_t t = t0 + (lane >> 4);
      const int e = e0 + (lane & 15);
      if (t < T && e < E) {
        float r = v[0];
        if (round_bf16) r = __bfloat162float(__float2bfloat16_rn(r));
        if (bias) r += bias[e];
        if (round_bf16 && bias) r = __bfloat162float(__float2bfloat16_rn(r));
        if (logits) logits[t * E + e] = r;
        const float gv = apply_sigmoid ? 1.0f / (1.0f + expf(-r)) : r;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i == (e0 >> 4)) picks[i] = gv;
      }
    }
    if (raw_sel != nullptr) {
      // top-k of the token's gate values inside its 16-lane half of the warp: descending value, ties to the lower
      // expert id, NaN never wins (the rules of topk_kernel)
      const int64_t t = t0 + (lane >> 4);
      for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = 16 * i + (lane & 15);
          if (e < E && (picks[i] > best || (picks[i] == best && e < best_e))) { best = picks[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
          if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = j;          // all-NaN row: keep indices in range
        if ((lane & 15) == 0 && t < T) {
          raw_sel[t * k + j] = best_e;
          gate[t * k + j] = best;
        }
        if ((best_e & 15) == (lane & 15)) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (i == (best_e >> 4)) picks[i] = -INFINITY;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------ router weight gradient
// dW_sel[e,:] = sum over the slots i of expert e of c_i * x[token_i,:], c_i = d gate * sigmoid' of the slot.
// One block per 64-slot segment of an expert (numbered like the 64-row tiles of the sorted slot list), 256
// threads x 4 columns per pass over D; the segment sums go to the workspace and a second kernel adds the
// segments of each expert in order: no atomics, bit-reproducible.
constexpr int kRwSeg = 64;
constexpr int kRwMaxBlocks = 320;          // blocks of the token-major variant (two per SM, at most this many)
constexpr size_t kRwSmemLimit = 200 * 1024;

__device__ __forceinline__ bool find_segment(const int32_t* off, int E, int64_t idx, int& e, int& beg, int& end) {
  int64_t before = 0;
  for (int x = 0; x < E; ++x) {
    const int b = off[x], en = off[x + 1];
    const int ns = (en - b + kRwSeg - 1) / kRwSeg;
    if (idx < before + ns) {
      e = x;
      beg = b + static_cast<int>(idx - before) * kRwSeg;
      end = min(beg + kRwSeg, en);
      return true;
    }
    before += ns;
  }
  return false;
}

template <typename TX>
__global__ void __launch_bounds__(256) router_dw_partial_kernel(const TX* __restrict__ x, int64_t x_stride, int64_t T, int D,
                                                                const float* __restrict__ dgate,
                                                                const float* __restrict__ gate, int apply_sigmoid,
                                                                const int32_t* __restrict__ token_index,
                                                                const int32_t* __restrict__ slot_index,
                                                                const int32_t* __restrict__ offsets, int E,
                                                                float* __restrict__ partials, int vec) {
  __shared__ int s_seg[3];
  __shared__ int s_row[kRwSeg];
  __shared__ float s_c[kRwSeg];
  if (threadIdx.x == 0) {
    int e = -1, beg = 0, end = 0;
    if (!find_segment(offsets, E, blockIdx.x, e, beg, end)) e = -1;
    s_seg[0] = e; s_seg[1] = beg; s_seg[2] = end;
  }
  __syncthreads();
  const int e = s_seg[0], beg = s_seg[1], end = s_seg[2];
  if (e < 0) return;
  const int n = end - beg;
  if (threadIdx.x < n) {
    const int i = beg + threadIdx.x;
    const int slot = slot_index[i];
    const int tok = token_index[i];
    const float g = gate[slot];
    const float c = apply_sigmoid ? (dgate[slot] * (1.f - g)) * g : dgate[slot];
    s_row[threadIdx.x] = (tok >= 0 && tok < T) ? tok : -1;
    s_c[threadIdx.x] = c;
  }
  __syncthreads();
  float* out = partials + static_cast<int64_t>(blockIdx.x) * D;
  for (int d = threadIdx.x * 4; d < D; d += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int r = 0; r < n; ++r) {
      const int tok = s_row[r];
      if (tok < 0) continue;
      const float4 v = ldg4<TX>(x + static_cast<int64_t>(tok) * x_stride + d, vec != 0, D - d);
      const float c = s_c[r];
      acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
    }
    if (vec && d + 3 < D) {        // vec implies D % 4 == 0: every partial row starts on a 16-byte boundary
      *reinterpret_cast<float4*>(out + d) = acc;
    } else {
      const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
      for (int j = 0; j < 4 && d + j < D; ++j) out[d + j] = a4[j];
    }
  }
}

__global__ void router_dw_reduce_kernel(const float* __restrict__ partials, const int32_t* __restrict__ offsets, int E,
                                        int D, float* __restrict__ dw) {
  __shared__ int s_first, s_count;
  const int e = blockIdx.y;
  if (threadIdx.x == 0) {
    int first = 0;
    for (int x = 0; x < e; ++x) first += (offsets[x + 1] - offsets[x] + kRwSeg - 1) / kRwSeg;
    s_first = first;
    s_count = (offsets[e + 1] - offsets[e] + kRwSeg - 1) / kRwSeg;
  }
  __syncthreads();
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float acc = 0.f;
  const float* p = partials + static_cast<int64_t>(s_first) * D + d;
  for (int s = 0; s < s_count; ++s) acc += p[static_cast<int64_t>(s) * D];
  dw[static_cast<int64_t>(e) * D + d] = acc;
}

// The same gradient, token-major, for routers whose whole [E,D] gradient fits in shared memory: a block walks a
// contiguous range of tokens, reads every x row once and adds c_j * x[t,:] into the rows of its k experts (a thread
// owns four columns of all E rows, so there is nothing to synchronise); the per-block results are summed in block
// order by a second kernel.  Reads x once instead of k times.
template <typename TX>
__global__ void __launch_bounds__(256) router_dw_token_kernel(const TX* __restrict__ x, int64_t x_stride, int64_t T, int D,
                                                              const float* __restrict__ dgate,
                                                              const float* __restrict__ gate, int apply_sigmoid,
                                                              const int32_t* __restrict__ raw_sel, int k, int E, int tpb,
                                                              float* __restrict__ partials) {
  extern __shared__ __align__(16) float s_acc[];      // [E][D], then tpb*k coefficients and expert ids
  float* s_c = s_acc + static_cast<size_t>(E) * D;
  int* s_e = reinterpret_cast<int*>(s_c + tpb * k);
  const int64_t t_beg = static_cast<int64_t>(blockIdx.x) * tpb;
  const int nt = static_cast<int>(min(static_cast<int64_t>(tpb), T - t_beg));
  for (int i = threadIdx.x * 4; i < E * D; i += 1024) *reinterpret_cast<float4*>(s_acc + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = threadIdx.x; i < nt * k; i += 256) {
    const int64_t s = t_beg * k + i;
    const float g = gate[s];
    const int e = raw_sel[s];
    s_c[i] = (e >= 0 && e < E) ? (apply_sigmoid ? (dgate[s] * (1.f - g)) * g : dgate[s]) : 0.f;
    s_e[i] = (e >= 0 && e < E) ? e : 0;
  }
  __syncthreads();
  for (int d = threadIdx.x * 4; d < D; d += 1024) {
    int t = 0;
    for (; t + 4 <= nt; t += 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ldg4<TX>(x + (t_beg + t + u) * x_stride + d, true, 4);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        for (int j = 0; j < k; ++j) {
          const float c = s_c[(t + u) * k + j];
          float4* a = reinterpret_cast<float4*>(s_acc + static_cast<size_t>(s_e[(t + u) * k + j]) * D + d);
          float4 o = *a;
          o.x = fmaf(c, v[u].x, o.x); o.y = fmaf(c, v[u].y, o.y); o.z = fmaf(c, v[u].z, o.z); o.w = fmaf(c, v[u].w, o.w);
          *a = o;
        }
      }
    }
    for (; t < nt; ++t) {
      const float4 v = ldg4<TX>(x + (t_beg + t) * x_stride + d, true, 4);
      for (int j = 0; j < k; ++j) {
        const float c = s_c[t * k + j];
        float4* a = reinterpret_cast<float4*>(s_acc + static_cast<size_t>(s_e[t * k + j]) * D + d);
        float4 o = *a;
        o.x = fmaf(c, v.x, o.x); o.y = fmaf(c, v.y, o.y); o.z = fmaf(c, v.z, o.z); o.w = fmaf(c, v.w, o.w);
        *a = o;
      }
    }
  }
  __syncthreads();
  float* out = partials + static_cast<size_t>(blockIdx.x) * E * D;
  for (int i = threadIdx.x * 4; i < E * D; i += 1024)
    *reinterpret_cast<float4*>(out + i) = *reinterpret_cast<const float4*>(s_acc + i);
}

// Block (32, 8): 32 column quads x 8 slices of the per-block results; a slice adds its contiguous range of blocks in
// order, then the eight slice sums are added in slice order.
__global__ void __launch_bounds__(256) router_dw_block_reduce_kernel(const float* __restrict__ partials, int nb, int64_t n,
                                                                     float* __restrict__ dw) {
  __shared__ float4 s_part[8][32];
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x) * 4;
  const int per = (nb + 7) / 8;
  const int b0 = threadIdx.y * per, b1 = min(nb, b0 + per);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i < n) {
#pragma unroll 4
    for (int b = b0; b < b1; ++b) {
      const float4 v = *reinterpret_cast<const float4*>(partials + static_cast<int64_t>(b) * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  s_part[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && i < n) {
#pragma unroll
    for (int sl = 1; sl < 8; ++sl) {
      const float4 v = s_part[sl][threadIdx.x];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(dw + i) = acc;
  }
}

// ------------------------------------------------------------------------------------ combine + router term
// y[t,:] = sum_j res[t*k+j,:]  +  sum_j c[t,j] * w_sel[raw_sel[t,j],:]      (j ascending, rows first)
template <typename TR, typename TW, typename TY>
__global__ void combine_router_kernel(const TR* __restrict__ res, int64_t res_stride, const int32_t* __restrict__ row_index,
                                      int64_t T, int k, int N,
                                      const float* __restrict__ dgate, const float* __restrict__ gate,
                                      int apply_sigmoid, const int32_t* __restrict__ raw_sel,
                                      const TW* __restrict__ w_sel, int E, TY* __restrict__ y, int64_t y_stride, int vec) {
  const int nq = (N + 3) / 4;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * nq) return;
  const int64_t t = idx / nq;
  const int n0 = static_cast<int>(idx - t * nq) * 4;
  const int valid = N - n0;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int j = 0; j < k; ++j) {
    const int64_t rr = row_index ? row_index[t * k + j] : t * k + j;
    const float4 v = ldg4<TR>(res + rr * res_stride + n0, vec != 0, valid);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
#pragma unroll 4
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const int e = raw_sel[s];
    if (e < 0 || e >= E) continue;
    const float g = gate[s];
    const float c = apply_sigmoid ? (dgate[s] * (1.f - g)) * g : dgate[s];
    const float4 v = ldg4<TW>(w_sel + static_cast<int64_t>(e) * N + n0, vec != 0, valid);
    acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
  }
  TY* dst = y + t * y_stride + n0;
  const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
  if (vec && valid >= 4) {
    if constexpr (sizeof(TY) == 4) {
      *reinterpret_cast<float4*>(dst) = acc;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  } else {
    for (int j = 0; j < 4 && j < valid; ++j) {
      if constexpr (sizeof(TY) == 4) dst[j] = a4[j];
      else dst[j] = __float2bfloat16_rn(a4[j]);
    }
  }
}

// The same for N % 512 == 0 and 16-byte aligned rows: a warp owns 512 columns of a token, lane l the column quads
// 4l + 128q (q = 0..3).  The per-slot scalars (row, expert, gate, gate gradient) are fetched once per 16 columns instead
// of once per 4, and 4k row loads are in flight per lane.  Per element the sums run in the same order.
template <typename TR, typename TW, typename TY>
__global__ void __launch_bounds__(256) combine_router512_kernel(const TR* __restrict__ res, int64_t res_stride,
                                         const int32_t* __restrict__ row_index, int64_t T, int k, int N,
                                         const float* __restrict__ dgate, const float* __restrict__ gate,
                                         int apply_sigmoid, const int32_t* __restrict__ raw_sel,
                                         const TW* __restrict__ w_sel, int E, TY* __restrict__ y, int64_t y_stride) {
  const int lane = threadIdx.x & 31;
  const int nb = N / 512;
  const int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= T * nb) return;
  const int64_t t = wid / nb;
  const int n0 = static_cast<int>(wid - t * nb) * 512 + 4 * lane;
  float4 acc[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
  for (int j = 0; j < k; ++j) {
    const int64_t rr = row_index ? row_index[t * k + j] : t * k + j;
    const TR* r = res + rr * res_stride + n0;
    float4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = ldg4<TR>(r + 128 * q, true, 4);
#pragma unroll
    for (int q = 0; q < 4; ++q) { acc[q].x += v[q].x; acc[q].y += v[q].y; acc[q].z += v[q].z; acc[q].w += v[q].w; }
  }
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const int e = raw_sel[s];
    if (e < 0 || e >= E) continue;
    const float g = gate[s];
    const float c = apply_sigmoid ? (dgate[s] * (1.f - g)) * g : dgate[s];
    const TW* wr = w_sel + static_cast<int64_t>(e) * N + n0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 v = ldg4<TW>(wr + 128 * q, true, 4);
      acc[q].x = fmaf(c, v.x, acc[q].x); acc[q].y = fmaf(c, v.y, acc[q].y);
      acc[q].z = fmaf(c, v.z, acc[q].z); acc[q].w = fmaf(c, v.w, acc[q].w);
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    TY* dst = y + t * y_stride + n0 + 128 * q;
    if constexpr (sizeof(TY) == 4) {
      *reinterpret_cast<float4*>(dst) = acc[q];
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc[q].x, acc[q].y), hi = __floats2bfloat162_rn(acc[q].z, acc[q].w);
      *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TX, typename TW>
int launch_logits(const void* x, int64_t x_stride, int64_t T, int D, const void* w, int E, const float* bias, int round_bf16,
                  float* logits, int vec, cudaStream_t stream, int k = 0, int apply_sigmoid = 0, int32_t* raw_sel = nullptr,
                  float* gate = nullptr) {
  const TX* xp = reinterpret_cast<const TX*>(x);
  const TW* wp = reinterpret_cast<const TW*>(w);
  const size_t smem = static_cast<size_t>((E + 15) / 16 * 16) * D * sizeof(float);
  if (vec && E <= 64 && smem <= kRwSmemLimit) {
    const int64_t pairs = (T + 1) / 2;
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    int64_t grid = (pairs + 7) / 8;
    if (grid > static_cast<int64_t>(per_sm) * sm_count()) grid = static_cast<int64_t>(per_sm) * sm_count();
    AMOE_CUDA(cudaFuncSetAttribute(router_logits_smem_kernel<TX, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem)));
    router_logits_smem_kernel<TX, TW><<<static_cast<unsigned>(grid), 256, smem, stream>>>(xp, x_stride, T, D, wp, E, bias,
                                                                                          round_bf16, logits, k, apply_sigmoid,
                                                                                          raw_sel, gate);
    AMOE_LAUNCH_CHECK("router_logits_smem");
    return AMOE_OK;
  }
  if (raw_sel != nullptr) return AMOE_ERR_UNSUPPORTED;      // the fused select needs the shared-memory variant
#define AMOE_RL(EQ)                                                                                              \
  do {                                                                                                           \
    constexpr int kTok = 2 * (128 / EQ);                                                                         \
    dim3 grid(static_cast<unsigned>((T + kTok - 1) / kTok), static_cast<unsigned>((E + 4 * EQ - 1) / (4 * EQ))); \
    router_logits_kernel<TX, TW, EQ><<<grid, 128, 0, stream>>>(xp, x_stride, T, D, wp, E, bias, round_bf16, logits, vec); \
  } while (0)
  if (E <= 4) AMOE_RL(1);
  else if (E <= 8) AMOE_RL(2);
  else if (E <= 16) AMOE_RL(4);
  else if (E <= 32) AMOE_RL(8);
  else AMOE_RL(16);
#undef AMOE_RL
  AMOE_LAUNCH_CHECK("router_logits");
  return AMOE_OK;
}

}  // namespace
}  // namespace amoe

using namespace amoe;

extern "C" {

int amoe_router_logits(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const void* w,
                       int32_t w_dtype, int32_t E, const float* bias, int32_t round_bf16, float* logits,
                       amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && w && logits, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && D > 0 && E > 0 && E <= 65535 * 64, AMOE_ERR_BAD_SHAPE);
  const int xs = x_dtype == AMOE_F32 ? 4 : 2, wsz = w_dtype == AMOE_F32 ? 4 : 2;
  const int vec = al16(x) && al16(w) && (x_stride * xs) % 16 == 0 && (static_cast<int64_t>(D) * wsz) % 16 == 0 && D % 4 == 0;
  if (x_dtype == AMOE_F32 && w_dtype == AMOE_F32)
    return launch_logits<float, float>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream);
  if (x_dtype == AMOE_BF16 && w_dtype == AMOE_BF16)
    return launch_logits<__nv_bfloat16, __nv_bfloat16>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream);
  if (x_dtype == AMOE_BF16 && w_dtype == AMOE_F32)
    return launch_logits<__nv_bfloat16, float>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream);
  if (x_dtype == AMOE_F32 && w_dtype == AMOE_BF16)
    return launch_logits<float, __nv_bfloat16>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream);
  return AMOE_ERR_BAD_DTYPE;
}

int amoe_router_select(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const void* w,
                       int32_t w_dtype, int32_t E, const float* bias, int32_t round_bf16, int32_t k, int32_t apply_sigmoid,
                       float* logits, int32_t* raw_sel, float* gate, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && w && raw_sel && gate, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && D > 0 && E > 0 && k > 0 && k <= E, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(E <= 64, AMOE_ERR_UNSUPPORTED);
  const int xs = x_dtype == AMOE_F32 ? 4 : 2, wsz = w_dtype == AMOE_F32 ? 4 : 2;
  const int vec = al16(x) && al16(w) && (x_stride * xs) % 16 == 0 && (static_cast<int64_t>(D) * wsz) % 16 == 0 && D % 4 == 0;
  AMOE_REQUIRE(vec, AMOE_ERR_UNSUPPORTED);
  if (x_dtype == AMOE_F32 && w_dtype == AMOE_F32)
    return launch_logits<float, float>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream, k, apply_sigmoid, raw_sel, gate);
  if (x_dtype == AMOE_BF16 && w_dtype == AMOE_BF16)
    return launch_logits<__nv_bfloat16, __nv_bfloat16>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream, k,
                                                       apply_sigmoid, raw_sel, gate);
  if (x_dtype == AMOE_BF16 && w_dtype == AMOE_F32)
    return launch_logits<__nv_bfloat16, float>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream, k, apply_sigmoid,
                                               raw_sel, gate);
  if (x_dtype == AMOE_F32 && w_dtype == AMOE_BF16)
    return launch_logits<float, __nv_bfloat16>(x, x_stride, T, D, w, E, bias, round_bf16, logits, vec, stream, k, apply_sigmoid,
                                               raw_sel, gate);
  return AMOE_ERR_BAD_DTYPE;
}

size_t amoe_router_backward_w_workspace_bytes(int64_t P, int32_t E, int32_t D) {
  if (P <= 0 || E <= 0 || D <= 0) return 0;
  const size_t by_segment = static_cast<size_t>(P / kRwSeg + E) * D * sizeof(float);
  const size_t by_block = static_cast<size_t>(kRwMaxBlocks) * E * D * sizeof(float);
  return by_segment > by_block ? by_segment : by_block;
}

int amoe_router_backward_w(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const float* dgate,
                           const float* gate, int32_t apply_sigmoid, const int32_t* token_index,
                           const int32_t* slot_index, const int32_t* expert_offsets, const int32_t* raw_sel, int64_t P,
                           int32_t E, float* dw_sel, void* workspace, size_t workspace_bytes, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && dgate && gate && token_index && slot_index && expert_offsets && dw_sel, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && D > 0 && P > 0 && E > 0 && E <= 65535 && P < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(workspace && workspace_bytes >= amoe_router_backward_w_workspace_bytes(P, E, D) && al16(workspace),
               AMOE_ERR_WORKSPACE);
  const int xs = x_dtype == AMOE_F32 ? 4 : 2;
  const int vec = al16(x) && (x_stride * xs) % 16 == 0 && D % 4 == 0;
  float* partials = reinterpret_cast<float*>(workspace);
  // token-major variant: the whole gradient in shared memory, x read once (needs the flat slot order t*k+j of
  // dgate/gate/raw_sel, which is what token_index/slot_index describe when P = T*k)
  const int k = static_cast<int>(P / T);
  if (raw_sel != nullptr && vec && static_cast<int64_t>(k) * T == P) {
    const int per_sm = static_cast<size_t>(E) * D * sizeof(float) <= 100 * 1024 ? 2 : 1;
    int nb = per_sm * sm_count() < kRwMaxBlocks ? per_sm * sm_count() : kRwMaxBlocks;
    if (nb > T) nb = static_cast<int>(T);
    const int tpb = static_cast<int>((T + nb - 1) / nb);
    nb = static_cast<int>((T + tpb - 1) / tpb);
    const size_t smem = (static_cast<size_t>(E) * D + static_cast<size_t>(tpb) * k * 2) * sizeof(float);
    if (smem <= kRwSmemLimit) {
      if (x_dtype == AMOE_F32) {
        AMOE_CUDA(cudaFuncSetAttribute(router_dw_token_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        router_dw_token_kernel<float><<<nb, 256, smem, stream>>>(reinterpret_cast<const float*>(x), x_stride, T, D, dgate, gate,
                                                                 apply_sigmoid, raw_sel, k, E, tpb, partials);
      } else if (x_dtype == AMOE_BF16) {
        AMOE_CUDA(cudaFuncSetAttribute(router_dw_token_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        router_dw_token_kernel<__nv_bfloat16><<<nb, 256, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), x_stride, T, D,
                                                                         dgate, gate, apply_sigmoid, raw_sel, k, E, tpb, partials);
      } else {
        return AMOE_ERR_BAD_DTYPE;
      }
      AMOE_LAUNCH_CHECK("router_dw_token");
      const int64_t n = static_cast<int64_t>(E) * D;
      router_dw_block_reduce_kernel<<<static_cast<unsigned>((n / 4 + 31) / 32), dim3(32, 8), 0, stream>>>(partials, nb, n, dw_sel);
      AMOE_LAUNCH_CHECK("router_dw_block_reduce");
      return AMOE_OK;
    }
  }
  const unsigned blocks = static_cast<unsigned>(P / kRwSeg + E);
  if (x_dtype == AMOE_F32)
    router_dw_partial_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), x_stride, T, D, dgate, gate,
                                                                apply_sigmoid, token_index, slot_index, expert_offsets, E,
                                                                partials, vec && D % 4 == 0);
  else if (x_dtype == AMOE_BF16)
    router_dw_partial_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), x_stride, T,
                                                                        D, dgate, gate, apply_sigmoid, token_index, slot_index,
                                                                        expert_offsets, E, partials, vec && D % 4 == 0);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("router_dw_partial");
  dim3 rg(static_cast<unsigned>((D + 255) / 256), static_cast<unsigned>(E));
  router_dw_reduce_kernel<<<rg, 256, 0, stream>>>(partials, expert_offsets, E, D, dw_sel);
  AMOE_LAUNCH_CHECK("router_dw_reduce");
  return AMOE_OK;
}

int amoe_combine_router(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, int64_t T,
                        int32_t k, int32_t N,
                        const float* dgate, const float* gate, int32_t apply_sigmoid, const int32_t* raw_sel,
                        const void* w_sel, int32_t w_dtype, int32_t E, void* y, int32_t y_dtype, int64_t y_stride,
                        amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(res && dgate && gate && raw_sel && w_sel && y, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && k > 0 && N > 0 && E > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(res_dtype == y_dtype && (w_dtype == AMOE_F32 || w_dtype == res_dtype), AMOE_ERR_BAD_DTYPE);
  const int rs = res_dtype == AMOE_F32 ? 4 : 2, wsz = w_dtype == AMOE_F32 ? 4 : 2;
  const int vec = (N % 4 == 0) && al16(res) && al16(y) && al16(w_sel) && (res_stride * rs) % 16 == 0 && (y_stride * rs) % 16 == 0 &&
                  (static_cast<int64_t>(N) * wsz) % 16 == 0;
  const int64_t n = T * ((N + 3) / 4);
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  const bool wide = vec && N % 512 == 0;
  const unsigned wblocks = static_cast<unsigned>((T * (N / 512 > 0 ? N / 512 : 1) * 32 + 255) / 256);
#define AMOE_CR(TR, TW)                                                                                               \
  if (wide)                                                                                                           \
    combine_router512_kernel<TR, TW, TR><<<wblocks, 256, 0, stream>>>(reinterpret_cast<const TR*>(res), res_stride, row_index, T, k, \
                                                                      N, dgate, gate, apply_sigmoid, raw_sel,        \
                                                                      reinterpret_cast<const TW*>(w_sel), E,          \
                                                                      reinterpret_cast<TR*>(y), y_stride);            \
  else                                                                                                                \
  combine_router_kernel<TR, TW, TR><<<blocks, 256, 0, stream>>>(reinterpret_cast<const TR*>(res), res_stride, row_index, T, k, N, dgate, \
                                                                gate, apply_sigmoid, raw_sel, reinterpret_cast<const TW*>(w_sel), \
                                                                E, reinterpret_cast<TR*>(y), y_stride, vec)
  if (res_dtype == AMOE_F32 && w_dtype == AMOE_F32) AMOE_CR(float, float);
  else if (res_dtype == AMOE_BF16 && w_dtype == AMOE_BF16) AMOE_CR(__nv_bfloat16, __nv_bfloat16);
  else if (res_dtype == AMOE_BF16 && w_dtype == AMOE_F32) AMOE_CR(__nv_bfloat16, float);
  else return AMOE_ERR_BAD_DTYPE;
#undef AMOE_CR
  AMOE_LAUNCH_CHECK("combine_router");
  return AMOE_OK;
}

}  // extern "C"
