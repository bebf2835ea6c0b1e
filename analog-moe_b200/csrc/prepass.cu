// Weight pre-pass (column maxima, weight modifier, bf16 hi/lo operand layouts) and row abs-max.
#include "common.cuh"

namespace amoe {
namespace {

// colmax[e,n] = max_k |W[e,k,n]|.  Block = 32 columns x 8 k-lanes over a slice of K; the slices meet
// through an integer atomic max on the bit patterns of the (non-negative) floats, which is exact
// and order-independent.  colmax must be zero-filled before the launch.
// With `colsum`/`colsq` given ([slices,E,N] doubles) the same pass also leaves each slice's sum and sum of squares
// per column: the statistics of the Gaussian weight clipping, summed later in slice order (no atomics).
constexpr int kColmaxSlice = 128;
__global__ void colmax_kernel(const void* __restrict__ w, int dtype, int E, int K, int N, int64_t se, int64_t sk,
                              int64_t sn, float* __restrict__ colmax, double* __restrict__ colsum,
                              double* __restrict__ colsq) {
  __shared__ float red[8][33];
  __shared__ double red_s[8][33], red_q[8][33];
  const int e = blockIdx.y;
  const int n = blockIdx.x * 32 + threadIdx.x;
  const int kb = blockIdx.z * kColmaxSlice;
  const int ke = min(K, kb + kColmaxSlice);
  float m = 0.f;
  double sum = 0.0, sq = 0.0;
  if (n < N) {
    for (int k = kb + threadIdx.y; k < ke; k += 8) {
      const float v = load_elem(w, dtype, e * se + k * sk + n * sn);
      m = fmaxf(m, fabsf(v));
      if (colsum) { sum += v; sq += static_cast<double>(v) * v; }
    }
  }
  red[threadIdx.y][threadIdx.x] = m;
  if (colsum) { red_s[threadIdx.y][threadIdx.x] = sum; red_q[threadIdx.y][threadIdx.x] = sq; }
  __syncthreads();
  if (threadIdx.y == 0 && n < N) {
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i][threadIdx.x]);
    if (m == m) atomicMax(reinterpret_cast<int*>(colmax) + static_cast<int64_t>(e) * N + n, __float_as_int(m));
    else colmax[static_cast<int64_t>(e) * N + n] = m;   // NaN weights: propagate
    if (colsum) {
      for (int i = 1; i < 8; ++i) { sum += red_s[i][threadIdx.x]; sq += red_q[i][threadIdx.x]; }
      const int64_t o = (static_cast<int64_t>(blockIdx.z) * E + e) * N + n;
      colsum[o] = sum;
      colsq[o] = sq;
    }
  }
}

// Clip bounds, one block per expert: bound[e,n] = min(sigma * std, fixed) with the unbiased standard deviation of
// the column (per_channel) or of the whole expert, and colmax[e,n] = min(colmax[e,n], bound[e,n]) - the column
// maximum of the clipped weights.  sigma <= 0: bound = fixed.
__global__ void __launch_bounds__(256) clip_bounds_kernel(const double* __restrict__ colsum, const double* __restrict__ colsq,
                                                          int slices, int E, int K, int N, float sigma, int per_channel,
                                                          float fixed, float* __restrict__ colmax,
                                                          float* __restrict__ bound) {
  __shared__ double s_sum[256], s_sq[256];
  const int e = blockIdx.x;
  double tsum = 0.0, tsq = 0.0;
  if (sigma > 0.f) {
    for (int n = threadIdx.x; n < N; n += 256) {
      double a = 0.0, b = 0.0;
      for (int sl = 0; sl < slices; ++sl) {
        const int64_t o = (static_cast<int64_t>(sl) * E + e) * N + n;
        a += colsum[o];
        b += colsq[o];
      }
      if (per_channel) {
        const double var = K > 1 ? (b - a * a / K) / (K - 1) : 0.0;
        float bd = sigma * static_cast<float>(sqrt(var > 0.0 ? var : 0.0));
        if (fixed > 0.f) bd = fminf(bd, fixed);
        const int64_t i = static_cast<int64_t>(e) * N + n;
        bound[i] = bd;
        colmax[i] = fminf(colmax[i], bd);
      } else {
        tsum += a;
        tsq += b;
      }
    }
  }
  if (sigma > 0.f && per_channel) return;
  float bd = fixed;
  if (sigma > 0.f) {
    s_sum[threadIdx.x] = tsum;
    s_sq[threadIdx.x] = tsq;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {        // fixed tree: the same result on every run
      if (threadIdx.x < o) { s_sum[threadIdx.x] += s_sum[threadIdx.x + o]; s_sq[threadIdx.x] += s_sq[threadIdx.x + o]; }
      __syncthreads();
    }
    const double cnt = static_cast<double>(K) * N;
    const double var = cnt > 1 ? (s_sq[0] - s_sum[0] * s_sum[0] / cnt) / (cnt - 1) : 0.0;
    bd = sigma * static_cast<float>(sqrt(var > 0.0 ? var : 0.0));
    if (fixed > 0.f) bd = fminf(bd, fixed);
  }
  for (int n = threadIdx.x; n < N; n += 256) {
    const int64_t i = static_cast<int64_t>(e) * N + n;
    bound[i] = bd;
    colmax[i] = fminf(colmax[i], bd);
  }
}

// One block per expert: expmax[e] = max_n colmax[e,n], then the output scales (per column or per expert) and
// their correctly rounded reciprocals.
__global__ void __launch_bounds__(256) scales_kernel(const float* __restrict__ colmax, int N, int per_channel,
                                                     float* __restrict__ expmax, float* __restrict__ out,
                                                     float* __restrict__ inv) {
  __shared__ float red[8];
  __shared__ float s_max;
  const int e = blockIdx.x;
  const float* cm = colmax + static_cast<int64_t>(e) * N;
  float m = 0.f;
  for (int n = threadIdx.x; n < N; n += 256) m = fmaxf(m, cm[n]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    expmax[e] = m;
    s_max = m;
  }
  __syncthreads();
  const float em = s_max;
  for (int n = threadIdx.x; n < N; n += 256) {
    const float s = per_channel ? cm[n] : em;
    const int64_t i = static_cast<int64_t>(e) * N + n;
    if (out) out[i] = s;
    if (inv) inv[i] = s > 0.f ? __frcp_rn(s) : 0.f;
  }
}

struct PrepassDev {
  const void* w; int dtype; int E, K, N; int64_t se, sk, sn;
  const float* colmax; const float* expmax;
  int noise_per_channel; float noise_std; float n_states;  // n_states<=0: no discretisation
  uint64_t seed; uint32_t offset; const long long* step_dev; int expert_base;
  float* w_out;
  const float* bound;   // [E,N] clip bound, or NULL
  void* w_clip_out;     // clamped weights in the layout and type of w (normally w itself), or NULL
  __nv_bfloat16 *fwd_hi, *fwd_lo, *bwd_hi, *bwd_lo;
  int Npad, Kpad, Kpad2, Npad2;
  int f16;              // the prepared copies hold IEEE fp16 (saturating at +-65504) instead of bf16; no lo terms
};

constexpr int kTK = 32, kTN = 128;

__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack2_f16(float a, float b) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint32_t pack2_op(float a, float b, int f16) { return f16 ? pack2_f16(a, b) : pack2_bf16(a, b); }

// Block (32,8): tile of 32 k-rows x 128 n-columns of expert blockIdx.z.  Loads, the modifier and the
// natural-orientation copy work on four consecutive columns per thread (16-byte loads, 8-byte bf16
// stores); the transposed copy goes through shared memory and leaves as 16-byte stores of eight
// consecutive k.
__global__ void __launch_bounds__(256) transform_kernel(PrepassDev p) {
  __shared__ float tile[kTK][kTN + 1];
  const int e = blockIdx.z;
  const int k0 = blockIdx.y * kTK, n0 = blockIdx.x * kTN;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int n = n0 + tx * 4;
  const bool vec_in = p.dtype == AMOE_F32 && p.sn == 1 && (p.sk % 4 == 0) && (p.se % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.w) & 15u) == 0) && n + 3 < p.N;
  const uint32_t off = p.offset + (p.step_dev ? static_cast<uint32_t>(*p.step_dev) * 8u : 0u);
  for (int r = ty; r < kTK; r += 8) {
    const int k = k0 + r;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k < p.K && n < p.N) {
      float z[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.noise_std > 0.f) {
        const float4 zz = philox_normal4_inline(p.seed, off, kStreamWeightNoise, static_cast<uint32_t>((p.expert_base + e) * p.K + k),
                                                static_cast<uint32_t>(n >> 2));
        z[0] = zz.x; z[1] = zz.y; z[2] = zz.z; z[3] = zz.w;
      }
      float x[4] = {0.f, 0.f, 0.f, 0.f};
      if (vec_in) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.w) + e * p.se + k * p.sk + n));
        x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) x[j] = load_elem(p.w, p.dtype, e * p.se + k * p.sk + (n + j) * p.sn);
      }
      if (p.bound) {
        // Gaussian / fixed-value weight clipping first: everything below sees the clipped weights, and they are
        // written back in place
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) {
            const float bd = p.bound[static_cast<int64_t>(e) * p.N + n + j];
            x[j] = fminf(fmaxf(x[j], -bd), bd);
            if (p.w_clip_out) store_elem(p.w_clip_out, p.dtype, e * p.se + k * p.sk + (n + j) * p.sn, x[j]);
          }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n + j < p.N) {
          float xv = x[j];
          const float s = p.noise_per_channel ? p.colmax[static_cast<int64_t>(e) * p.N + n + j] : p.expmax[e];
          if (p.n_states > 0.f) {
            const float res = __fdiv_rn(s, p.n_states);
            if (res > 0.f) {
              xv = rintf(__fdiv_rn(xv, res)) * res;
              xv = fminf(fmaxf(xv, -s), s);
            }
          }
          if (p.noise_std > 0.f) xv = xv + (p.noise_std * s) * z[j];
          v[j] = xv;
        }
      }
      if (p.w_out) {
        float* dst = p.w_out + (static_cast<int64_t>(e) * p.K + k) * p.N + n;
        if (n + 3 < p.N && (p.N % 4 == 0)) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else
          for (int j = 0; j < 4; ++j)
            if (n + j < p.N) dst[j] = v[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) tile[r][tx * 4 + j] = v[j];
    // natural orientation: row k, n contiguous (Npad2 is a multiple of 64, so whole quads fit)
    if (p.bwd_hi && k < p.Kpad2 && n < p.Npad2) {
      const uint32_t h0 = pack2_op(v[0], v[1], p.f16), h1 = pack2_op(v[2], v[3], p.f16);
      const int64_t o = (static_cast<int64_t>(e) * p.Kpad2 + k) * p.Npad2 + n;
      *reinterpret_cast<uint2*>(p.bwd_hi + o) = make_uint2(h0, h1);
      if (p.bwd_lo) {
        const uint32_t l0 = pack2_bf16(v[0] - __uint_as_float(h0 << 16), v[1] - __uint_as_float(h0 & 0xffff0000u));
        const uint32_t l1 = pack2_bf16(v[2] - __uint_as_float(h1 << 16), v[3] - __uint_as_float(h1 & 0xffff0000u));
        *reinterpret_cast<uint2*>(p.bwd_lo + o) = make_uint2(l0, l1);
      }
    }
  }
  __syncthreads();
  if (p.fwd_hi) {
    // transposed orientation: row n, k contiguous.  256 threads: column = tid/2, 16 k-values each
    // (Kpad is a multiple of 64, so the 32-row tile lies inside the padded extent or entirely outside).
    const int tid = ty * 32 + tx;
    const int c = tid >> 1, half = tid & 1;
    const int nn = n0 + c;
    const int kb = k0 + half * 16;
    if (nn < p.Npad && kb < p.Kpad) {
      uint32_t h[8], l[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a = tile[half * 16 + 2 * i][c], b2 = tile[half * 16 + 2 * i + 1][c];
        h[i] = pack2_op(a, b2, p.f16);
        l[i] = pack2_bf16(a - __uint_as_float(h[i] << 16), b2 - __uint_as_float(h[i] & 0xffff0000u));
      }
      const int64_t o = (static_cast<int64_t>(e) * p.Npad + nn) * p.Kpad + kb;
      uint4* dh = reinterpret_cast<uint4*>(p.fwd_hi + o);
      dh[0] = make_uint4(h[0], h[1], h[2], h[3]);
      dh[1] = make_uint4(h[4], h[5], h[6], h[7]);
      if (p.fwd_lo) {
        uint4* dl = reinterpret_cast<uint4*>(p.fwd_lo + o);
        dl[0] = make_uint4(l[0], l[1], l[2], l[3]);
        dl[1] = make_uint4(l[4], l[5], l[6], l[7]);
      }
    }
  }
}

// max|x| of a whole tensor through an integer atomic max on the bit patterns (non-negative floats order like
// integers; NaNs are skipped).  `out` must be zero before the launch.
template <typename T>
__global__ void tensor_absmax_kernel(const T* __restrict__ x, int64_t rows, int K, int64_t stride,
                                     const int32_t* __restrict__ n_rows_dev, float* __restrict__ out, int vec) {
  int64_t n = rows;
  if (n_rows_dev != nullptr) n = min(static_cast<int64_t>(max(*n_rows_dev, 0)), rows);
  float m = 0.f;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthr = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    // rows are contiguous and 16-byte aligned: one flat stream of 16-byte pieces, four in flight per thread
    constexpr int per = 16 / sizeof(T);
    const uint4* p = reinterpret_cast<const uint4*>(x);
    const int64_t total = n * K / per;
    for (int64_t i = tid; i < total; i += 4 * nthr) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (i + u * nthr < total) ? __ldg(p + i + u * nthr) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (sizeof(T) == 4) {
            const float f = fabsf(__uint_as_float(w[j]));
            if (f == f) m = fmaxf(m, f);
          } else {
            const float a = fabsf(__uint_as_float(w[j] << 16)), b2 = fabsf(__uint_as_float(w[j] & 0xffff0000u));
            if (a == a) m = fmaxf(m, a);
            if (b2 == b2) m = fmaxf(m, b2);
          }
        }
      }
    }
  } else {
    const int lane = threadIdx.x & 31;
    for (int64_t r = tid >> 5; r < n; r += nthr >> 5) {
      const T* row = x + r * stride;
      for (int k = lane; k < K; k += 32) {
        const float v = fabsf(to_f32<T>(row[k]));
        if (v == v) m = fmaxf(m, v);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
}

template <typename T>
__global__ void row_absmax_kernel(const T* __restrict__ x, int64_t R, int K, int64_t stride, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (r >= R) return;
  const T* row = x + r * stride;
  float m = 0.f;
  for (int k = lane; k < K; k += 32) m = fmaxf(m, fabsf(to_f32<T>(row[k])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) out[r] = m;
}

}  // namespace
}  // namespace amoe

using namespace amoe;

extern "C" {

size_t amoe_weight_prepass_workspace_bytes(int32_t E, int32_t K, int32_t N) {
  if (E <= 0 || N <= 0) return 0;
  (void)K;
  return (static_cast<size_t>(E) * N + E) * sizeof(float);
}

// With clipping: the same plus bound [E,N] floats and two [slices,E,N] double arrays (8-byte aligned).
size_t amoe_weight_prepass_clip_workspace_bytes(int32_t E, int32_t K, int32_t N) {
  if (E <= 0 || N <= 0 || K <= 0) return 0;
  const size_t en = static_cast<size_t>(E) * N;
  const size_t head = ((2 * en + E) * sizeof(float) + 7) & ~static_cast<size_t>(7);
  const size_t slices = (static_cast<size_t>(K) + kColmaxSlice - 1) / kColmaxSlice;
  return head + 2 * slices * en * sizeof(double);
}

void amoe_prepared_dims(int32_t K, int32_t N, int32_t dims[4]) {
  dims[0] = round_up(N, 16); dims[1] = round_up(K, 64); dims[2] = round_up(K, 16); dims[3] = round_up(N, 64);
}

int amoe_weight_prepass(const amoe_weight_prepass_args* a, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(a != nullptr && a->w != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->E > 0 && a->K > 0 && a->N > 0 && a->E <= 65535, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->w_dtype == AMOE_F32 || a->w_dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE(a->workspace && a->workspace_bytes >= amoe_weight_prepass_workspace_bytes(a->E, a->K, a->N),
               AMOE_ERR_WORKSPACE);
  AMOE_REQUIRE(!(a->fwd_lo && !a->fwd_hi) && !(a->bwd_lo && !a->bwd_hi), AMOE_ERR_NULL_POINTER);
  const bool clip = a->clip_sigma > 0.f || a->clip_fixed > 0.f;
  const size_t en = static_cast<size_t>(a->E) * a->N;
  const int slices = (a->K + kColmaxSlice - 1) / kColmaxSlice;
  float* colmax = reinterpret_cast<float*>(a->workspace);
  float* expmax = colmax + en;
  float* bound = nullptr;
  double* colsum = nullptr;
  double* colsq = nullptr;
  if (clip) {
    AMOE_REQUIRE(a->workspace_bytes >= amoe_weight_prepass_clip_workspace_bytes(a->E, a->K, a->N), AMOE_ERR_WORKSPACE);
    AMOE_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 7u) == 0, AMOE_ERR_WORKSPACE);
    bound = expmax + a->E;
    if (a->clip_sigma > 0.f) {
      const size_t head = ((2 * en + a->E) * sizeof(float) + 7) & ~static_cast<size_t>(7);
      colsum = reinterpret_cast<double*>(reinterpret_cast<uint8_t*>(a->workspace) + head);
      colsq = colsum + static_cast<size_t>(slices) * en;
    }
  }
  AMOE_CUDA(cudaMemsetAsync(colmax, 0, en * sizeof(float), stream));
  colmax_kernel<<<dim3((a->N + 31) / 32, a->E, slices), dim3(32, 8), 0, stream>>>(
      a->w, a->w_dtype, a->E, a->K, a->N, a->w_stride_e, a->w_stride_k, a->w_stride_n, colmax, colsum, colsq);
  AMOE_LAUNCH_CHECK("colmax");
  if (clip) {
    clip_bounds_kernel<<<a->E, 256, 0, stream>>>(colsum, colsq, slices, a->E, a->K, a->N, a->clip_sigma,
                                                 a->clip_per_channel, a->clip_fixed, colmax, bound);
    AMOE_LAUNCH_CHECK("clip_bounds");
  }
  scales_kernel<<<a->E, 256, 0, stream>>>(colmax, a->N, a->per_channel_scale, expmax, a->col_scale, a->col_inv_scale);
  AMOE_LAUNCH_CHECK("scales");
  if (a->w_out || a->fwd_hi || a->bwd_hi || (clip && a->w_clip_out)) {
    PrepassDev p;
    p.bound = bound; p.w_clip_out = clip ? a->w_clip_out : nullptr;
    p.w = a->w; p.dtype = a->w_dtype; p.E = a->E; p.K = a->K; p.N = a->N;
    p.se = a->w_stride_e; p.sk = a->w_stride_k; p.sn = a->w_stride_n;
    p.colmax = colmax; p.expmax = expmax;
    p.noise_per_channel = a->noise_per_channel; p.noise_std = a->noise_std;
    p.n_states = a->discretize_res > 0.f ? fmaxf(a->discretize_res, 1.0f / a->discretize_res) : -1.f;
    p.seed = a->seed; p.offset = a->offset; p.step_dev = a->step_dev; p.expert_base = a->expert_base;
    p.w_out = a->w_out;
    p.fwd_hi = reinterpret_cast<__nv_bfloat16*>(a->fwd_hi); p.fwd_lo = reinterpret_cast<__nv_bfloat16*>(a->fwd_lo);
    p.bwd_hi = reinterpret_cast<__nv_bfloat16*>(a->bwd_hi); p.bwd_lo = reinterpret_cast<__nv_bfloat16*>(a->bwd_lo);
    p.f16 = a->prepared_f16;
    AMOE_REQUIRE(!p.f16 || (!a->fwd_lo && !a->bwd_lo), AMOE_ERR_UNSUPPORTED);
    p.Npad = round_up(a->N, 16); p.Kpad = round_up(a->K, 64);
    p.Kpad2 = round_up(a->K, 16); p.Npad2 = round_up(a->N, 64);
    const int kext = p.Kpad, next = p.Npad2;  // Kpad >= Kpad2, Npad2 >= Npad
    dim3 grid((next + kTN - 1) / kTN, (kext + kTK - 1) / kTK, a->E);
    AMOE_REQUIRE(grid.y <= 65535, AMOE_ERR_BAD_SHAPE);
    transform_kernel<<<grid, dim3(32, 8), 0, stream>>>(p);
    AMOE_LAUNCH_CHECK("transform");
  }
  return AMOE_OK;
}

int amoe_tensor_absmax(const void* x, int32_t dtype, int64_t rows, int32_t K, int64_t stride, const int32_t* n_rows_dev,
                       float* absmax, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && absmax, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(rows > 0 && K > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_CUDA(cudaMemsetAsync(absmax, 0, sizeof(float), stream));
  const unsigned blocks = static_cast<unsigned>(sm_count()) * 8u;
  const int esz = dtype == AMOE_F32 ? 4 : 2;
  const int vec = stride == K && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (static_cast<int64_t>(K) * esz) % 16 == 0;
  if (dtype == AMOE_F32)
    tensor_absmax_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), rows, K, stride, n_rows_dev, absmax,
                                                            vec);
  else if (dtype == AMOE_BF16)
    tensor_absmax_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), rows, K, stride,
                                                                    n_rows_dev, absmax, vec);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("tensor_absmax");
  return AMOE_OK;
}

int amoe_row_absmax(const void* x, int32_t dtype, int64_t R, int32_t K, int64_t stride, float* absmax,
                    amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && absmax, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(R > 0 && K > 0, AMOE_ERR_BAD_SHAPE);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((R * 32 + threads - 1) / threads);
  if (dtype == AMOE_F32)
    row_absmax_kernel<float><<<blocks, threads, 0, stream>>>(reinterpret_cast<const float*>(x), R, K, stride, absmax);
  else if (dtype == AMOE_BF16)
    row_absmax_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), R, K,
                                                                     stride, absmax);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("row_absmax");
  return AMOE_OK;
}

}  // extern "C"
