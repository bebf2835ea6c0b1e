// Reductions around the CVMM (combine over k, gate gradient, input-range gradient, per-expert
// std) and the expert-parallel pack/unpack helpers.  All HBM-bound streaming kernels.
#include <mutex>

#include "common.cuh"

namespace amoe {
namespace {

// Four consecutive elements starting at p (16-byte / 8-byte / 4-byte vector load when `vec`, else element by
// element with `valid` of them inside the row; the rest read as zero).
template <typename T>
__device__ __forceinline__ void ld4(const T* p, bool vec, int valid, float o[4]) {
  if (vec) {
    if constexpr (sizeof(T) == 4) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(p));
      o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
    } else {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
      o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
      o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] = c < valid ? to_f32<T>(p[c]) : 0.f;
  }
}
// Four int8 codes packed in a word as floats, without integer->float conversions: flipping each byte's top bit turns
// the code c into the unsigned byte c + 128; dropped into the low byte of 0x4B400000 (= 1.5 * 2^23) that is the float
// 1.5 * 2^23 + c + 128 exactly, and one subtraction leaves c.
__device__ __forceinline__ void codes4_to_float(uint32_t u, float o[4]) {
  const uint32_t x = u ^ 0x80808080u;
  o[0] = __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7650)) - 12583040.f;
  o[1] = __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7651)) - 12583040.f;
  o[2] = __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7652)) - 12583040.f;
  o[3] = __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7653)) - 12583040.f;
}
__device__ __forceinline__ void ld4_codes(const int8_t* p, bool vec, int valid, float o[4]) {
  if (vec) {
    codes4_to_float(__ldg(reinterpret_cast<const uint32_t*>(p)), o);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] = c < valid ? static_cast<float>(p[c]) : 0.f;
  }
}
template <typename T>
__device__ __forceinline__ void st4(T* p, bool vec, int valid, const float v[4]) {
  if (vec) {
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (c < valid) {
        if constexpr (sizeof(T) == 4) p[c] = v[c];
        else p[c] = __float2bfloat16_rn(v[c]);
      }
  }
}

// y[t,n] = sum_j w[t*k+j] * res[row(t*k+j), n]; thread per (t, 4 columns); j ascending.
template <typename TR, typename TY>
__global__ void combine_kernel(const TR* __restrict__ res, int64_t res_stride, const int32_t* __restrict__ row_index,
                               const float* __restrict__ w, int64_t T, int k, int N, TY* __restrict__ y,
                               int64_t y_stride, int vec) {
  const int nq = (N + 3) / 4;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * nq) return;
  const int64_t t = idx / nq;
  const int n0 = static_cast<int>(idx - t * nq) * 4;
  const int valid = N - n0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const float ws = w ? w[s] : 1.f;
    const int64_t rr = row_index ? row_index[s] : s;
    float v[4];
    ld4<TR>(res + rr * res_stride + n0, vec != 0, valid, v);
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[c] = w ? fmaf(ws, v[c], acc[c]) : acc[c] + v[c];
  }
  st4<TY>(y + t * y_stride + n0, vec != 0, valid, acc);
}

template <typename TY>
__global__ void combine_codes_kernel(const int8_t* __restrict__ codes, const float* __restrict__ col_scale,
                                     const int32_t* __restrict__ raw_sel, const float* __restrict__ row_mult,
                                     float step, const float* __restrict__ w, int64_t T, int k, int N,
                                     TY* __restrict__ y, int64_t y_stride, int vec,
                                     const int32_t* __restrict__ row_index) {
  const int nq = (N + 3) / 4;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * nq) return;
  const int64_t t = idx / nq;
  const int n0 = static_cast<int>(idx - t * nq) * 4;
  const int valid = N - n0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const float ws = w ? w[s] : 1.f;
    const int64_t rr = row_index ? row_index[s] : s;       // where the slot's row (codes, row_mult) is kept
    const float rm = row_mult ? row_mult[rr] : 1.f;
    const int e = raw_sel[s];
    float cd[4], cs[4];
    ld4_codes(codes + rr * N + n0, vec != 0, valid, cd);
    ld4<float>(col_scale + static_cast<int64_t>(e) * N + n0, vec != 0, valid, cs);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float v = __fmul_rn(__fmul_rn(__fmul_rn(cd[c], step), cs[c]), rm);   // the row value, rounded as the kernel rounds it
      acc[c] = fmaf(ws, v, acc[c]);
    }
  }
  st4<TY>(y + t * y_stride + n0, vec != 0, valid, acc);
}

// The same sum for rows of 16-byte aligned codes with N % 16 == 0: a thread owns 16 columns (one 16-byte load of
// codes per slot), which amortises the per-slot scalars; per element the arithmetic and its order are unchanged.
template <typename TY>
__global__ void combine_codes16_kernel(const int8_t* __restrict__ codes, const float* __restrict__ col_scale,
                                       const int32_t* __restrict__ raw_sel, const float* __restrict__ row_mult,
                                       float step, const float* __restrict__ w, int64_t T, int k, int N,
                                       TY* __restrict__ y, int64_t y_stride, const int32_t* __restrict__ row_index) {
  const int ng = N / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * ng) return;
  const int64_t t = idx / ng;
  const int n0 = static_cast<int>(idx - t * ng) * 16;
  float acc[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) acc[c] = 0.f;
#pragma unroll 2
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const float ws = w ? w[s] : 1.f;
    const int64_t rr = row_index ? row_index[s] : s;
    const float rm = row_mult ? row_mult[rr] : 1.f;
    const int e = raw_sel[s];
    const uint4 cd = __ldg(reinterpret_cast<const uint4*>(codes + rr * N + n0));
    const float4* csp = reinterpret_cast<const float4*>(col_scale + static_cast<int64_t>(e) * N + n0);
    const uint32_t cw[4] = {cd.x, cd.y, cd.z, cd.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 cs = __ldg(csp + q);
      const float csv[4] = {cs.x, cs.y, cs.z, cs.w};
      float cdq[4];
      codes4_to_float(cw[q], cdq);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float cdv = cdq[c];
        const float v = __fmul_rn(__fmul_rn(__fmul_rn(cdv, step), csv[c]), rm);
        acc[4 * q + c] = fmaf(ws, v, acc[4 * q + c]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) st4<TY>(y + t * y_stride + n0 + 4 * q, true, 4, acc + 4 * q);
}

// The same sum with N % 512 == 0: a warp owns 512 columns of a token, lane l the four column quads 4l + 128q (q = 0..3),
// so that every load and store of a warp covers contiguous memory (128 bytes of codes, 512 bytes of column scales
// and of the result per instruction) while the per-slot scalars are still fetched once per 16 columns.  Per element the
// arithmetic and its order are unchanged.
template <typename TY>
__global__ void __launch_bounds__(256) combine_codes512_kernel(const int8_t* __restrict__ codes, const float* __restrict__ col_scale,
                                        const int32_t* __restrict__ raw_sel, const float* __restrict__ row_mult,
                                        float step, const float* __restrict__ w, int64_t T, int k, int N,
                                        TY* __restrict__ y, int64_t y_stride, const int32_t* __restrict__ row_index) {
  const int lane = threadIdx.x & 31;
  const int nb = N / 512;
  const int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= T * nb) return;
  const int64_t t = wid / nb;
  const int n0 = static_cast<int>(wid - t * nb) * 512 + 4 * lane;
  float acc[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) acc[c] = 0.f;
#pragma unroll 2
  for (int j = 0; j < k; ++j) {
    const int64_t s = t * k + j;
    const float ws = w ? w[s] : 1.f;
    const int64_t rr = row_index ? row_index[s] : s;
    const float rm = row_mult ? row_mult[rr] : 1.f;
    const int e = raw_sel[s];
    const int8_t* cp = codes + rr * N + n0;
    const float* csp = col_scale + static_cast<int64_t>(e) * N + n0;
    uint32_t cw[4];
    float4 cs[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      cw[q] = __ldg(reinterpret_cast<const uint32_t*>(cp + 128 * q));
      cs[q] = __ldg(reinterpret_cast<const float4*>(csp + 128 * q));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float csv[4] = {cs[q].x, cs[q].y, cs[q].z, cs[q].w};
      float cdq[4];
      codes4_to_float(cw[q], cdq);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float v = __fmul_rn(__fmul_rn(__fmul_rn(cdq[c], step), csv[c]), rm);
        acc[4 * q + c] = fmaf(ws, v, acc[4 * q + c]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) st4<TY>(y + t * y_stride + n0 + 128 * q, true, 4, acc + 4 * q);
}

// d[s] = res[row(s),:] . g[s/k,:]; one warp per slot; lane l walks the column quads l, l+32, ... and adds their
// four products in column order into one accumulator (the same order in the kernel below, so that rows rebuilt
// from codes give the same bits as materialised rows).
template <typename TR, typename TG>
__global__ void row_dot_kernel(const TR* __restrict__ res, int64_t res_stride, const int32_t* __restrict__ row_index,
                               const TG* __restrict__ g, int64_t g_stride, int64_t P, int k, int N,
                               float* __restrict__ d, int vec) {
  const int lane = threadIdx.x & 31;
  const int64_t s = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (s >= P) return;
  const TR* r = res + (row_index ? static_cast<int64_t>(row_index[s]) : s) * res_stride;
  const TG* gr = g + (s / k) * g_stride;
  const int nq = (N + 3) / 4;
  float acc = 0.f;
#pragma unroll 4
  for (int q = lane; q < nq; q += 32) {
    float a[4], b[4];
    ld4<TR>(r + 4 * q, vec != 0, N - 4 * q, a);
    ld4<TG>(gr + 4 * q, vec != 0, N - 4 * q, b);
#pragma unroll
    for (int c = 0; c < 4; ++c) acc = fmaf(a[c], b[c], acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) d[s] = acc;
}

// d[s] = sum_n ((code*step)*col_scale[e,n])*row_scale[s] * g[s/k,n]; one warp per slot, order as above.
template <typename TG>
__global__ void row_dot_codes_kernel(const int8_t* __restrict__ codes, const float* __restrict__ col_scale,
                                     const int32_t* __restrict__ row_expert, const float* __restrict__ row_scale,
                                     float step, const TG* __restrict__ g, int64_t g_stride, int64_t P, int k, int N,
                                     float* __restrict__ d, int vec, const int32_t* __restrict__ row_index) {
  const int lane = threadIdx.x & 31;
  const int64_t s = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (s >= P) return;
  const int64_t rr = row_index ? row_index[s] : s;        // row of codes / row_scale; row_expert stays by slot
  const int8_t* r = codes + rr * N;
  const float* cs = col_scale + static_cast<int64_t>(row_expert[s]) * N;
  const float rs = row_scale ? row_scale[rr] : 1.f;
  const TG* gr = g + (s / k) * g_stride;
  const int nq = (N + 3) / 4;
  float acc = 0.f;
#pragma unroll 4
  for (int q = lane; q < nq; q += 32) {
    float cd[4], sc[4], b[4];
    ld4_codes(r + 4 * q, vec != 0, N - 4 * q, cd);
    ld4<float>(cs + 4 * q, vec != 0, N - 4 * q, sc);
    ld4<TG>(gr + 4 * q, vec != 0, N - 4 * q, b);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float v = __fmul_rn(__fmul_rn(__fmul_rn(cd[c], step), sc[c]), rs);
      acc = fmaf(v, b[c], acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) d[s] = acc;
}

// The same dot products with one warp per TOKEN: the gradient row is loaded once for the token's k slots (it was the
// largest stream of the slot-per-warp kernel above) and stays in registers, 1024 columns at a time.  Per slot the
// lane's products are added in the same order as above, so the results are bit-identical.  k <= KMAX.
template <typename TG, int KMAX>
__global__ void __launch_bounds__(256) row_dot_codes_token_kernel(
    const int8_t* __restrict__ codes, const float* __restrict__ col_scale, const int32_t* __restrict__ row_expert,
    const float* __restrict__ row_scale, float step, const TG* __restrict__ g, int64_t g_stride, int64_t T, int k, int N,
    float* __restrict__ d, const int32_t* __restrict__ row_index) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  const TG* gr = g + t * g_stride;
  const int nq = N / 4;
  float acc[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) acc[j] = 0.f;
  for (int q0 = 0; q0 < nq; q0 += 256) {
    float b[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = q0 + lane + 32 * i;
      if (q < nq) ld4<TG>(gr + 4 * q, true, 4, b[i]);
    }
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < k) {
        const int64_t s = t * k + j;
        const int64_t rr = row_index ? row_index[s] : s;
        const int8_t* r = codes + rr * N;
        const float* cs = col_scale + static_cast<int64_t>(row_expert[s]) * N;
        const float rs = row_scale ? row_scale[rr] : 1.f;
        uint32_t cw[8];
        float4 sc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int q = q0 + lane + 32 * i;
          if (q < nq) {
            cw[i] = __ldg(reinterpret_cast<const uint32_t*>(r + 4 * q));
            sc[i] = __ldg(reinterpret_cast<const float4*>(cs + 4 * q));
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int q = q0 + lane + 32 * i;
          if (q < nq) {
            float cd[4];
            codes4_to_float(cw[i], cd);
            const float scv[4] = {sc[i].x, sc[i].y, sc[i].z, sc[i].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float v = __fmul_rn(__fmul_rn(__fmul_rn(cd[c], step), scv[c]), rs);
              acc[j] = fmaf(v, b[i][c], acc[j]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k) {
      float a = acc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane == 0) d[t * k + j] = a;
    }
  }
}

// One CTA of 256 threads per expert: fixed-order (thread-strided, butterfly inside each warp, then across the
// eight warps) sum of the expert's slot gradients.
__global__ void __launch_bounds__(256) ir_grad_reduce_kernel(const float* __restrict__ slot_grad,
                                                             const int32_t* __restrict__ offsets,
                                                             const float* __restrict__ input_range, int E, float decay,
                                                             float min_pct,
                                                             const unsigned long long* __restrict__ keep_count,
                                                             double total, const long long* __restrict__ total_rows_dev,
                                                             int cols, float* __restrict__ out) {
  __shared__ float red[8];
  const int e = blockIdx.x;
  const int beg = offsets[e], end = offsets[e + 1];
  float acc = 0.f;
  for (int i = beg + threadIdx.x; i < end; i += 256) acc += slot_grad[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    acc = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) acc += red[w];
    if (decay > 0.f && keep_count != nullptr) {
      // denominator: a device counter of rows (times the row length) when given, else the host's value, else the
      // rows this slot list holds
      double tot = total;
      if (total_rows_dev != nullptr) tot = static_cast<double>(*total_rows_dev) * cols;
      else if (!(tot > 0.0)) tot = static_cast<double>(offsets[E]) * cols;
      const float pct = static_cast<float>(static_cast<double>(*keep_count) / tot);
      if (pct > min_pct) acc += (decay * input_range[e]) * static_cast<float>(end - beg);
    }
    out[e] = acc;
  }
}

// ws layout: double sum[E], double sq[E]
template <typename T>
__global__ void std_sum_kernel(const T* __restrict__ x, int64_t stride, int K, int64_t x_rows,
                               const int32_t* __restrict__ x_row, const int32_t* __restrict__ offsets, int E, int pass,
                               const double* __restrict__ mean, double* __restrict__ accum, int32_t* status) {
  // one warp per sorted position; block-level reduce per expert would need segmenting, so use one
  // double atomic per warp (count of atomics = P, all on E addresses; this runs a handful of times
  // per training run).
  const int lane = threadIdx.x & 31;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t P = offsets[E];
  if (i >= P) return;
  // expert of position i by binary search in offsets
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offsets[mid] <= i) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int64_t src = x_row[i];
  if (src < 0 || src >= x_rows) {   // recorded and skipped, never dereferenced
    if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 40, static_cast<int>(i), static_cast<int>(src));
    return;
  }
  const T* row = x + src * stride;
  double acc = 0.0;
  if (pass == 0) {
    for (int k = lane; k < K; k += 32) acc += static_cast<double>(to_f32<T>(row[k]));
  } else {
    const double mu = mean[e];
    for (int k = lane; k < K; k += 32) {
      double dlt = static_cast<double>(to_f32<T>(row[k])) - mu;
      acc += dlt * dlt;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) atomicAdd(accum + e, acc);
}

__global__ void std_mean_kernel(const double* __restrict__ sum, const int32_t* __restrict__ offsets, int E, int K,
                                double* __restrict__ mean) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const double cnt = static_cast<double>(offsets[e + 1] - offsets[e]) * K;
  mean[e] = sum[e] / cnt;   // 0/0 = NaN for an expert without rows
}

__global__ void std_final_kernel(const double* __restrict__ sq, const int32_t* __restrict__ offsets, int E, int K,
                                 float* __restrict__ out) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const double cnt = static_cast<double>(offsets[e + 1] - offsets[e]) * K;
  out[e] = cnt > 0 ? static_cast<float>(sqrt(sq[e] / (cnt - 1.0))) : __int_as_float(0x7fc00000);
}

// Gather rows in sorted order; optionally apply the DAC and emit int8 codes + per-row scale.
template <typename T>
__global__ void ep_pack_kernel(const T* __restrict__ x, int64_t stride, int K, const int32_t* __restrict__ src_row,
                               int src_div, const float* __restrict__ row_scale, int64_t P,
                               const float* __restrict__ ir, float inp_res, T* __restrict__ send_rows,
                               int8_t* __restrict__ send_codes, float* __restrict__ send_scale) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (i >= P) return;
  const int64_t sr = src_row[i];
  const T* row = x + (sr / src_div) * stride;
  if (send_codes) {
    const float r = ir[i];
    const float rr = __frcp_rn(r), rcp_res = quant_rcp(inp_res);
    for (int k = lane; k < K; k += 32) {
      float c = dac_code(to_f32<T>(row[k]), true, r, rr, false, 1.f, 1.f, inp_res, rcp_res);
      send_codes[i * K + k] = static_cast<int8_t>(c);
    }
    if (lane == 0) send_scale[i] = r;
  } else if (row_scale) {
    const float sc = row_scale[sr];
    for (int k = lane; k < K; k += 32) {
      if constexpr (sizeof(T) == 4) send_rows[i * K + k] = sc * row[k];
      else send_rows[i * K + k] = __float2bfloat16_rn(sc * __bfloat162float(row[k]));
    }
  } else {
    for (int k = lane; k < K; k += 32) send_rows[i * K + k] = row[k];
  }
}

__global__ void invert_index_kernel(const int32_t* __restrict__ idx, int64_t P, int32_t* __restrict__ inv) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const int32_t j = idx[i];
  if (j >= 0 && j < P) inv[j] = static_cast<int32_t>(i);
}

template <typename T>
__global__ void ep_unpack_kernel(const T* __restrict__ recv, int N, const int32_t* __restrict__ dst_row, int64_t P,
                                 T* __restrict__ out, int64_t out_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (i >= P) return;
  T* row = out + static_cast<int64_t>(dst_row[i]) * out_stride;
  for (int n = lane; n < N; n += 32) row[n] = recv[i * N + n];
}

// Scratch of amoe_expert_std_static: sum[E], sq[E], mean[E] in double precision for up to
// kStaticStdMaxExperts experts.  Lives in every CUDA context that loads the library (96 KiB).
constexpr int kStaticStdMaxExperts = 4096;
static __device__ __align__(256) double g_std_scratch[3 * kStaticStdMaxExperts];

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline unsigned blocks_for(int64_t threads, int per_block) {
  return static_cast<unsigned>((threads + per_block - 1) / per_block);
}

// The receive buffer of an expert-parallel rank holds, for source g = 0..G-1, that source's rows for local experts
// 0..El-1 in order: block (g, e) has recv_counts[g*El + e] rows.  Expert-sorted order is: for e, for g, block (g, e).
// local_order[sorted position] = row of the receive buffer; local_offsets[e] = first sorted position of expert e.
constexpr int kEpMaxBlocks = 4096;
__global__ void __launch_bounds__(256) ep_local_plan_kernel(const int32_t* __restrict__ recv_counts, int G, int El, int R,
                                                            int32_t* __restrict__ local_order,
                                                            int32_t* __restrict__ local_offsets) {
  __shared__ int s_recv_start[kEpMaxBlocks + 1];    // by receive order  (g major)
  __shared__ int s_sorted_start[kEpMaxBlocks];      // by receive order, value = start in sorted order
  const int nb = G * El;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int b = 0; b < nb; ++b) { s_recv_start[b] = acc; acc += recv_counts[b]; }
    s_recv_start[nb] = acc;
    acc = 0;
    for (int e = 0; e < El; ++e) {
      if (blockIdx.x == 0) local_offsets[e] = acc;
      for (int g = 0; g < G; ++g) { s_sorted_start[g * El + e] = acc; acc += recv_counts[g * El + e]; }
    }
    if (blockIdx.x == 0) local_offsets[El] = acc;
  }
  __syncthreads();
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < R; r += gridDim.x * blockDim.x) {
    int lo = 0, hi = nb;               // last block whose start is <= r (empty blocks share a start: take the last)
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_recv_start[mid] <= r) lo = mid; else hi = mid;
    }
    local_order[s_sorted_start[lo] + (r - s_recv_start[lo])] = r;
  }
}

}  // namespace
}  // namespace amoe

using namespace amoe;

extern "C" {

int amoe_combine(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, const float* w,
                 int64_t T, int32_t k, int32_t N, void* y, int32_t y_dtype, int64_t y_stride, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(res && y, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && k > 0 && N > 0, AMOE_ERR_BAD_SHAPE);
  const int64_t n = T * ((N + 3) / 4);
  const unsigned blocks = blocks_for(n, 256);
  const int vec = (N % 4 == 0) && (res_stride % 4 == 0) && (y_stride % 4 == 0) && al16(res) && al16(y);
  if (res_dtype == AMOE_F32 && y_dtype == AMOE_F32)
    combine_kernel<float, float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(res), res_stride, row_index, w, T, k,
                                                             N, reinterpret_cast<float*>(y), y_stride, vec);
  else if (res_dtype == AMOE_BF16 && y_dtype == AMOE_BF16)
    combine_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(res), res_stride, row_index, w, T, k, N, reinterpret_cast<__nv_bfloat16*>(y),
        y_stride, vec);
  else if (res_dtype == AMOE_F32 && y_dtype == AMOE_BF16)
    combine_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(res), res_stride, row_index, w, T, k, N, reinterpret_cast<__nv_bfloat16*>(y),
                                                                     y_stride, vec);
  else if (res_dtype == AMOE_BF16 && y_dtype == AMOE_F32)
    combine_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(res),
                                                                     res_stride, row_index, w, T, k, N,
                                                                     reinterpret_cast<float*>(y), y_stride, vec);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("combine");
  return AMOE_OK;
}

int amoe_combine_codes(const int8_t* codes, const float* col_scale, const int32_t* raw_sel, const float* row_mult,
                       float step, const float* w, int64_t T, int32_t k, int32_t N, void* y, int32_t y_dtype,
                       int64_t y_stride, const int32_t* row_index, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(codes && col_scale && raw_sel && y, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(T > 0 && k > 0 && N > 0, AMOE_ERR_BAD_SHAPE);
  const int64_t n = T * ((N + 3) / 4);
  const unsigned blocks = blocks_for(n, 256);
  const int vec = (N % 4 == 0) && (y_stride % 4 == 0) && al16(y) && al16(col_scale) && al16(codes);
  if (vec && N % 512 == 0 && (y_dtype == AMOE_F32 || y_dtype == AMOE_BF16)) {
    const unsigned b512 = blocks_for(T * (N / 512) * 32, 256);
    if (y_dtype == AMOE_F32)
      combine_codes512_kernel<float><<<b512, 256, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T, k, N,
                                                               reinterpret_cast<float*>(y), y_stride, row_index);
    else
      combine_codes512_kernel<__nv_bfloat16><<<b512, 256, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T, k, N,
                                                                       reinterpret_cast<__nv_bfloat16*>(y), y_stride, row_index);
    AMOE_LAUNCH_CHECK("combine_codes512");
    return AMOE_OK;
  }
  if (vec && N % 16 == 0 && (y_dtype == AMOE_F32 || y_dtype == AMOE_BF16)) {
    const unsigned b16 = blocks_for(T * (N / 16), 128);
    if (y_dtype == AMOE_F32)
      combine_codes16_kernel<float><<<b16, 128, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T, k, N,
                                                             reinterpret_cast<float*>(y), y_stride, row_index);
    else
      combine_codes16_kernel<__nv_bfloat16><<<b16, 128, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T, k, N,
                                                                     reinterpret_cast<__nv_bfloat16*>(y), y_stride, row_index);
    AMOE_LAUNCH_CHECK("combine_codes16");
    return AMOE_OK;
  }
  if (y_dtype == AMOE_F32)
    combine_codes_kernel<float><<<blocks, 256, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T, k, N,
                                                            reinterpret_cast<float*>(y), y_stride, vec, row_index);
  else if (y_dtype == AMOE_BF16)
    combine_codes_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(codes, col_scale, raw_sel, row_mult, step, w, T,
                                                                    k, N, reinterpret_cast<__nv_bfloat16*>(y),
                                                                    y_stride, vec, row_index);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("combine_codes");
  return AMOE_OK;
}

int amoe_row_dot(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, const void* g,
                 int32_t g_dtype, int64_t g_stride, int64_t P, int32_t k, int32_t N, float* d, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(res && g && d, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && k > 0 && N > 0, AMOE_ERR_BAD_SHAPE);
  const unsigned blocks = blocks_for(P * 32, 256);
  const int vec = (N % 4 == 0) && (res_stride % 4 == 0) && (g_stride % 4 == 0) && al16(res) && al16(g);
  if (res_dtype == AMOE_F32 && g_dtype == AMOE_F32)
    row_dot_kernel<float, float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(res), res_stride, row_index,
                                                             reinterpret_cast<const float*>(g), g_stride, P, k, N, d, vec);
  else if (res_dtype == AMOE_BF16 && g_dtype == AMOE_BF16)
    row_dot_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(res), res_stride, row_index, reinterpret_cast<const __nv_bfloat16*>(g), g_stride,
        P, k, N, d, vec);
  else if (res_dtype == AMOE_F32 && g_dtype == AMOE_BF16)
    row_dot_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(res), res_stride, row_index,
                                                                     reinterpret_cast<const __nv_bfloat16*>(g),
                                                                     g_stride, P, k, N, d, vec);
  else if (res_dtype == AMOE_BF16 && g_dtype == AMOE_F32)
    row_dot_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(res),
                                                                     res_stride, row_index, reinterpret_cast<const float*>(g),
                                                                     g_stride, P, k, N, d, vec);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("row_dot");
  return AMOE_OK;
}

int amoe_row_dot_codes(const int8_t* codes, const float* col_scale, const int32_t* row_expert, const float* row_scale,
                       float step, const void* g, int32_t g_dtype, int64_t g_stride, int64_t P, int32_t k, int32_t N,
                       float* d, const int32_t* row_index, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(codes && col_scale && row_expert && g && d, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && k > 0 && N > 0, AMOE_ERR_BAD_SHAPE);
  const unsigned blocks = blocks_for(P * 32, 256);
  const int vec = (N % 4 == 0) && (g_stride % 4 == 0) && al16(g) && al16(col_scale) && al16(codes);
  if (vec && k <= 8 && P % k == 0 && (g_dtype == AMOE_F32 || g_dtype == AMOE_BF16)) {
    // one warp per token (g_stride % 8 == 0 for bf16 rows: 8-byte loads)
    const int64_t T = P / k;
    const unsigned tb = blocks_for(T * 32, 256);
    if (g_dtype == AMOE_F32) {
      row_dot_codes_token_kernel<float, 8><<<tb, 256, 0, stream>>>(codes, col_scale, row_expert, row_scale, step,
                                                                   reinterpret_cast<const float*>(g), g_stride, T, k, N, d, row_index);
      AMOE_LAUNCH_CHECK("row_dot_codes_token");
      return AMOE_OK;
    }
    if (g_stride % 8 == 0) {
      row_dot_codes_token_kernel<__nv_bfloat16, 8><<<tb, 256, 0, stream>>>(
          codes, col_scale, row_expert, row_scale, step, reinterpret_cast<const __nv_bfloat16*>(g), g_stride, T, k, N, d,
          row_index);
      AMOE_LAUNCH_CHECK("row_dot_codes_token");
      return AMOE_OK;
    }
  }
  if (g_dtype == AMOE_F32)
    row_dot_codes_kernel<float><<<blocks, 256, 0, stream>>>(codes, col_scale, row_expert, row_scale, step,
                                                            reinterpret_cast<const float*>(g), g_stride, P, k, N, d, vec, row_index);
  else if (g_dtype == AMOE_BF16)
    row_dot_codes_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(codes, col_scale, row_expert, row_scale, step,
                                                                    reinterpret_cast<const __nv_bfloat16*>(g), g_stride,
                                                                    P, k, N, d, vec, row_index);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("row_dot_codes");
  return AMOE_OK;
}

int amoe_ir_grad_reduce(const float* ir_grad_slot, const int32_t* expert_offsets, const float* input_range, int32_t E,
                        float decay, float min_percentage, const unsigned long long* keep_count,
                        double total_elements, const long long* total_rows_dev, int32_t cols, float* out,
                        amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(ir_grad_slot && expert_offsets && out, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(E > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(!(decay > 0.f) || (keep_count && input_range), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!(decay > 0.f) || total_elements > 0 || cols > 0, AMOE_ERR_BAD_SHAPE);
  ir_grad_reduce_kernel<<<static_cast<unsigned>(E), 256, 0, stream>>>(
      ir_grad_slot, expert_offsets, input_range, E, decay, min_percentage, keep_count, total_elements, total_rows_dev,
      cols, out);
  AMOE_LAUNCH_CHECK("ir_grad_reduce");
  return AMOE_OK;
}

size_t amoe_expert_std_workspace_bytes(int32_t E) { return E > 0 ? static_cast<size_t>(E) * 3 * sizeof(double) : 0; }

int amoe_expert_std(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows, const int32_t* x_row,
                    const int32_t* expert_offsets, int64_t P, int32_t E, float* std_out, void* workspace,
                    size_t workspace_bytes, int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && x_row && expert_offsets && std_out, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && E > 0 && K > 0 && x_rows > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(dtype == AMOE_F32 || dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE(workspace && workspace_bytes >= amoe_expert_std_workspace_bytes(E), AMOE_ERR_WORKSPACE);
  double* sum = reinterpret_cast<double*>(workspace);
  double* sq = sum + E;
  double* mean = sq + E;
  AMOE_CUDA(cudaMemsetAsync(workspace, 0, static_cast<size_t>(E) * 2 * sizeof(double), stream));
  const unsigned blocks = blocks_for(P * 32, 256);
  const unsigned eb = blocks_for(E, 128);
  for (int pass = 0; pass < 2; ++pass) {
    if (dtype == AMOE_F32)
      std_sum_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), stride, K, x_rows, x_row,
                                                        expert_offsets, E, pass, mean, pass == 0 ? sum : sq, dev_status);
    else
      std_sum_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), stride, K,
                                                                x_rows, x_row, expert_offsets, E, pass, mean,
                                                                pass == 0 ? sum : sq, dev_status);
    AMOE_LAUNCH_CHECK("std_sum");
    if (pass == 0) {
      std_mean_kernel<<<eb, 128, 0, stream>>>(sum, expert_offsets, E, K, mean);
      AMOE_LAUNCH_CHECK("std_mean");
    }
  }
  std_final_kernel<<<eb, 128, 0, stream>>>(sq, expert_offsets, E, K, std_out);
  AMOE_LAUNCH_CHECK("std_final");
  return AMOE_OK;
}

int amoe_expert_std_static(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows,
                           const int32_t* x_row, const int32_t* expert_offsets, int64_t P, int32_t E, float* std_out,
                           int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && x_row && expert_offsets && std_out, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && E > 0 && K > 0 && x_rows > 0, AMOE_ERR_BAD_SHAPE);
  if (E > kStaticStdMaxExperts) {
    set_last_error("amoe_expert_std_static: more experts than the built-in scratch holds (4096)", cudaErrorInvalidValue);
    return AMOE_ERR_BAD_SHAPE;
  }
  AMOE_REQUIRE(dtype == AMOE_F32 || dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  // Device address of the scratch array, looked up once per device with that device current.
  // (In host code `g_std_scratch` is only a handle for the symbol, never a device pointer.)
  constexpr int kMaxDevices = 64;
  static double* scratch_of_device[kMaxDevices] = {nullptr};
  static std::mutex lookup_mutex;
  int dev = -1;
  AMOE_CUDA(cudaGetDevice(&dev));
  AMOE_REQUIRE(dev >= 0 && dev < kMaxDevices, AMOE_ERR_DEVICE);
  double* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(lookup_mutex);
    if (scratch_of_device[dev] == nullptr) {
      void* addr = nullptr;
      AMOE_CUDA(cudaGetSymbolAddress(&addr, g_std_scratch));
      scratch_of_device[dev] = static_cast<double*>(addr);
    }
    scratch = scratch_of_device[dev];
  }
  double* sum = scratch;
  double* sq = scratch + kStaticStdMaxExperts;
  double* mean = scratch + 2 * kStaticStdMaxExperts;
  // the array still holds the previous call's sums: clear the two accumulators
  AMOE_CUDA(cudaMemsetAsync(scratch, 0, static_cast<size_t>(2) * kStaticStdMaxExperts * sizeof(double), stream));
  const unsigned blocks = blocks_for(P * 32, 256);
  const unsigned eb = blocks_for(E, 128);
  for (int pass = 0; pass < 2; ++pass) {
    if (dtype == AMOE_F32)
      std_sum_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), stride, K, x_rows, x_row,
                                                        expert_offsets, E, pass, mean, pass == 0 ? sum : sq, dev_status);
    else
      std_sum_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), stride, K,
                                                                x_rows, x_row, expert_offsets, E, pass, mean,
                                                                pass == 0 ? sum : sq, dev_status);
    AMOE_LAUNCH_CHECK("std_sum");
    if (pass == 0) {
      std_mean_kernel<<<eb, 128, 0, stream>>>(sum, expert_offsets, E, K, mean);
      AMOE_LAUNCH_CHECK("std_mean");
    }
  }
  std_final_kernel<<<eb, 128, 0, stream>>>(sq, expert_offsets, E, K, std_out);
  AMOE_LAUNCH_CHECK("std_final");
  return AMOE_OK;
}

int amoe_ep_local_plan(const int32_t* recv_counts, int32_t G, int32_t El, int64_t R, int32_t* local_order,
                       int32_t* local_offsets, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(recv_counts && local_order && local_offsets, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(G > 0 && El > 0 && R >= 0 && G * El <= kEpMaxBlocks && R < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  const unsigned blocks = R > 0 ? blocks_for(R, 256) : 1u;
  ep_local_plan_kernel<<<blocks > 1024u ? 1024u : blocks, 256, 0, stream>>>(recv_counts, G, El, static_cast<int>(R), local_order,
                                                                           local_offsets);
  AMOE_LAUNCH_CHECK("ep_local_plan");
  return AMOE_OK;
}

int amoe_invert_index(const int32_t* idx, int64_t P, int32_t* inv, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(idx && inv, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0, AMOE_ERR_BAD_SHAPE);
  invert_index_kernel<<<blocks_for(P, 256), 256, 0, stream>>>(idx, P, inv);
  AMOE_LAUNCH_CHECK("invert_index");
  return AMOE_OK;
}

int amoe_ep_pack(const void* x, int32_t dtype, int64_t stride, int32_t K, const int32_t* src_row, int32_t src_div,
                 const float* row_scale, int64_t P, const float* ir, float inp_res, void* send_rows,
                 int8_t* send_codes, float* send_scale, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && src_row, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && K > 0, AMOE_ERR_BAD_SHAPE);
  if (src_div < 1) src_div = 1;
  AMOE_REQUIRE((send_codes != nullptr) != (send_rows != nullptr), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!send_codes || (ir && send_scale && inp_res > 0.f && inp_res >= 1.f / 127.5f), AMOE_ERR_UNSUPPORTED);
  const unsigned blocks = blocks_for(P * 32, 256);
  if (dtype == AMOE_F32)
    ep_pack_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(x), stride, K, src_row, src_div,
                                                      row_scale, P, ir,
                                                      inp_res, reinterpret_cast<float*>(send_rows), send_codes,
                                                      send_scale);
  else if (dtype == AMOE_BF16)
    ep_pack_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), stride, K,
                                                              src_row, src_div, row_scale, P, ir, inp_res,
                                                              reinterpret_cast<__nv_bfloat16*>(send_rows), send_codes,
                                                              send_scale);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("ep_pack");
  return AMOE_OK;
}

int amoe_ep_unpack(const void* recv_rows, int32_t dtype, int32_t N, const int32_t* dst_row, int64_t P, void* out,
                   int64_t out_stride, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(recv_rows && dst_row && out, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && N > 0, AMOE_ERR_BAD_SHAPE);
  const unsigned blocks = blocks_for(P * 32, 256);
  if (dtype == AMOE_F32)
    ep_unpack_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(recv_rows), N, dst_row, P,
                                                        reinterpret_cast<float*>(out), out_stride);
  else if (dtype == AMOE_BF16)
    ep_unpack_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(recv_rows), N,
                                                                dst_row, P, reinterpret_cast<__nv_bfloat16*>(out),
                                                                out_stride);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("ep_unpack");
  return AMOE_OK;
}

}  // extern "C"
