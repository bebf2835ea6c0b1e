// Weight pre-pass (column maxima, weight modifier, bf16 hi/lo operand layouts) and row abs-max.
#include "common.cuh"

namespace amoe {
namespace {

// colmax[e,n] = max_k |W[e,k,n]|.  Block = 32 columns x 8 k-lanes.
__global__ void colmax_kernel(const void* __restrict__ w, int dtype, int E, int K, int N, int64_t se, int64_t sk,
                              int64_t sn, float* __restrict__ colmax) {
  __shared__ float red[8][33];
  const int e = blockIdx.y;
  const int n = blockIdx.x * 32 + threadIdx.x;
  float m = 0.f;
  if (n < N) {
    for (int k = threadIdx.y; k < K; k += 8) m = fmaxf(m, fabsf(load_elem(w, dtype, e * se + k * sk + n * sn)));
  }
  red[threadIdx.y][threadIdx.x] = m;
  __syncthreads();
  if (threadIdx.y == 0 && n < N) {
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i][threadIdx.x]);
    colmax[static_cast<int64_t>(e) * N + n] = m;
  }
}

// expmax[e] = max_n colmax[e,n]; one block per expert.
__global__ void expmax_kernel(const float* __restrict__ colmax, int N, float* __restrict__ expmax) {
  __shared__ float red[32];
  const int e = blockIdx.x;
  float m = 0.f;
  for (int n = threadIdx.x; n < N; n += blockDim.x) m = fmaxf(m, colmax[static_cast<int64_t>(e) * N + n]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (threadIdx.x == 0) expmax[e] = m;
  }
}

__global__ void fill_scale_kernel(const float* __restrict__ colmax, const float* __restrict__ expmax, int E, int N,
                                  int per_channel, float* __restrict__ out, float* __restrict__ inv) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(E) * N) return;
  const float s = per_channel ? colmax[i] : expmax[i / N];
  if (out) out[i] = s;
  if (inv) inv[i] = s > 0.f ? __frcp_rn(s) : 0.f;
}

struct PrepassDev {
  const void* w; int dtype; int E, K, N; int64_t se, sk, sn;
  const float* colmax; const float* expmax;
  int noise_per_channel; float noise_std; float n_states;  // n_states<=0: no discretisation
  uint64_t seed; uint32_t offset; const long long* step_dev;
  float* w_out;
  __nv_bfloat16 *fwd_hi, *fwd_lo, *bwd_hi, *bwd_lo;
  int Npad, Kpad, Kpad2, Npad2;
};

constexpr int kTK = 32, kTN = 128;

// Block (32,8): tile of 32 k-rows x 128 n-columns of expert blockIdx.z.
__global__ void __launch_bounds__(256) transform_kernel(PrepassDev p) {
  __shared__ float tile[kTK][kTN + 1];
  const int e = blockIdx.z;
  const int k0 = blockIdx.y * kTK, n0 = blockIdx.x * kTN;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int n = n0 + tx * 4;
  for (int r = ty; r < kTK; r += 8) {
    const int k = k0 + r;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k < p.K && n < p.N) {
      float z[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.noise_std > 0.f) {
        const uint32_t off = p.offset + (p.step_dev ? static_cast<uint32_t>(*p.step_dev) * 8u : 0u);
        float4 zz = philox_normal4(p.seed, off, kStreamWeightNoise, static_cast<uint32_t>(e * p.K + k),
                                   static_cast<uint32_t>(n >> 2));
        z[0] = zz.x; z[1] = zz.y; z[2] = zz.z; z[3] = zz.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n + j < p.N) {
          float x = load_elem(p.w, p.dtype, e * p.se + k * p.sk + (n + j) * p.sn);
          float s = p.noise_per_channel ? p.colmax[static_cast<int64_t>(e) * p.N + n + j] : p.expmax[e];
          if (p.n_states > 0.f) {
            float res = __fdiv_rn(s, p.n_states);
            if (res > 0.f) {
              x = rintf(__fdiv_rn(x, res)) * res;
              x = fminf(fmaxf(x, -s), s);
            }
          }
          if (p.noise_std > 0.f) x = x + (p.noise_std * s) * z[j];
          v[j] = x;
        }
      }
      if (p.w_out) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) p.w_out[(static_cast<int64_t>(e) * p.K + k) * p.N + n + j] = v[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) tile[r][tx * 4 + j] = v[j];
    // natural orientation: row k, n contiguous
    if (p.bwd_hi && k < p.Kpad2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n + j < p.Npad2) {
          __nv_bfloat16 hi, lo;
          split_bf16(v[j], hi, lo);
          const int64_t o = (static_cast<int64_t>(e) * p.Kpad2 + k) * p.Npad2 + n + j;
          p.bwd_hi[o] = hi;
          if (p.bwd_lo) p.bwd_lo[o] = lo;
        }
      }
    }
  }
  __syncthreads();
  if (p.fwd_hi) {
    // transposed orientation: row n, k contiguous.  256 threads: column = tid/2, 16 k-values each.
    const int tid = ty * 32 + tx;
    const int c = tid >> 1, half = tid & 1;
    const int nn = n0 + c;
    if (nn < p.Npad) {
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int r = half * 16 + i;
        const int k = k0 + r;
        if (k < p.Kpad) {
          __nv_bfloat16 hi, lo;
          split_bf16(tile[r][c], hi, lo);
          const int64_t o = (static_cast<int64_t>(e) * p.Npad + nn) * p.Kpad + k;
          p.fwd_hi[o] = hi;
          if (p.fwd_lo) p.fwd_lo[o] = lo;
        }
      }
    }
  }
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
  float* colmax = reinterpret_cast<float*>(a->workspace);
  float* expmax = colmax + static_cast<size_t>(a->E) * a->N;
  colmax_kernel<<<dim3((a->N + 31) / 32, a->E), dim3(32, 8), 0, stream>>>(a->w, a->w_dtype, a->E, a->K, a->N,
                                                                          a->w_stride_e, a->w_stride_k,
                                                                          a->w_stride_n, colmax);
  AMOE_LAUNCH_CHECK("colmax");
  expmax_kernel<<<a->E, 256, 0, stream>>>(colmax, a->N, expmax);
  AMOE_LAUNCH_CHECK("expmax");
  if (a->col_scale || a->col_inv_scale) {
    const int64_t n = static_cast<int64_t>(a->E) * a->N;
    fill_scale_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(colmax, expmax, a->E, a->N,
                                                                                  a->per_channel_scale, a->col_scale,
                                                                                  a->col_inv_scale);
    AMOE_LAUNCH_CHECK("fill_scale");
  }
  if (a->w_out || a->fwd_hi || a->bwd_hi) {
    PrepassDev p;
    p.w = a->w; p.dtype = a->w_dtype; p.E = a->E; p.K = a->K; p.N = a->N;
    p.se = a->w_stride_e; p.sk = a->w_stride_k; p.sn = a->w_stride_n;
    p.colmax = colmax; p.expmax = expmax;
    p.noise_per_channel = a->noise_per_channel; p.noise_std = a->noise_std;
    p.n_states = a->discretize_res > 0.f ? fmaxf(a->discretize_res, 1.0f / a->discretize_res) : -1.f;
    p.seed = a->seed; p.offset = a->offset; p.step_dev = a->step_dev;
    p.w_out = a->w_out;
    p.fwd_hi = reinterpret_cast<__nv_bfloat16*>(a->fwd_hi); p.fwd_lo = reinterpret_cast<__nv_bfloat16*>(a->fwd_lo);
    p.bwd_hi = reinterpret_cast<__nv_bfloat16*>(a->bwd_hi); p.bwd_lo = reinterpret_cast<__nv_bfloat16*>(a->bwd_lo);
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
