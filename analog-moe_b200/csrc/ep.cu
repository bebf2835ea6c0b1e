// Device-driven expert-parallel exchange: the plan of one step (who sends how many rows where) is computed on the
// device from the all-gathered count matrix, and rows are written straight into the destination rank's buffer by
// plain stores over NVLink (peer pointers of a symmetric allocation).  Nothing here needs a value on the host, so
// the whole step can be captured in a CUDA graph.  No kernel waits on another rank: ordering between ranks comes
// from the collectives the caller places between these launches.
#include "common.cuh"

namespace amoe {
namespace {

constexpr int kEpMaxRanks = 64;
constexpr int kEpMaxBlocksDev = 4096;

// plan layout (int32): [0] R = rows this rank receives, [1] rows this rank sends (= its slot count),
// then four arrays of G: send_off (start of destination d's block in this rank's sorted slot list), off_in (start of
// this rank's block in destination d's receive buffer), recv_off (start of source s's block in this rank's receive
// buffer), back_off (start of this rank's block in source s's sorted slot list); then recv_counts [G, El].
__host__ __device__ inline int plan_ints(int G, int El) { return 2 + 4 * G + G * El; }

__global__ void ep_plan_kernel(const int32_t* __restrict__ gathered, int me, int G, int El, int32_t* __restrict__ plan) {
  __shared__ int tot[kEpMaxRanks * kEpMaxRanks];
  for (int i = threadIdx.x; i < G * G; i += blockDim.x) {
    int acc = 0;
    for (int e = 0; e < El; ++e) acc += gathered[i * El + e];
    tot[i] = acc;
  }
  for (int i = threadIdx.x; i < G * El; i += blockDim.x) {
    const int g = i / El, e = i - g * El;
    plan[2 + 4 * G + i] = gathered[(g * G + me) * El + e];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t* send_off = plan + 2;
    int32_t* off_in = send_off + G;
    int32_t* recv_off = off_in + G;
    int32_t* back_off = recv_off + G;
    int acc = 0;
    for (int d = 0; d < G; ++d) { send_off[d] = acc; acc += tot[me * G + d]; }
    plan[1] = acc;
    acc = 0;
    for (int s = 0; s < G; ++s) { recv_off[s] = acc; acc += tot[s * G + me]; }
    plan[0] = acc;
    for (int d = 0; d < G; ++d) {
      int a = 0;
      for (int s = 0; s < me; ++s) a += tot[s * G + d];
      off_in[d] = a;
    }
    for (int s = 0; s < G; ++s) {
      int a = 0;
      for (int d = 0; d < me; ++d) a += tot[s * G + d];
      back_off[s] = a;
    }
  }
}

// local_order / local_offsets as ep_local_plan_kernel, with the counts and R read from the plan.
__global__ void __launch_bounds__(256) ep_local_plan_dev_kernel(const int32_t* __restrict__ plan, int G, int El, int cap,
                                                                int32_t* __restrict__ local_order,
                                                                int32_t* __restrict__ local_offsets,
                                                                int32_t* __restrict__ status) {
  __shared__ int s_recv_start[kEpMaxBlocksDev + 1];
  __shared__ int s_sorted_start[kEpMaxBlocksDev];
  const int32_t* recv_counts = plan + 2 + 4 * G;
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
  if (plan[0] > cap && blockIdx.x == 0 && threadIdx.x == 0) report(status, AMOE_ERR_INDEX_RANGE, 50, plan[0], cap);
  const int R = min(plan[0], cap);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < R; r += gridDim.x * blockDim.x) {
    int lo = 0, hi = nb;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_recv_start[mid] <= r) lo = mid; else hi = mid;
    }
    // a position in the full permutation of plan[0] rows: it lies inside the array only if the plan fits the buffer
    const int pos = s_sorted_start[lo] + (r - s_recv_start[lo]);
    if (pos < cap) local_order[pos] = r;
  }
}

// Order in which the warps of a launch take the rows.  The slot list is sorted by expert, hence by destination rank,
// and the receive buffer by source rank: taken in order, every rank would write to rank 0 first, then to rank 1, ...,
// and each destination's NVLink ingress would serve all senders at once while the other links idle.  Warp w takes
// row (w mod kSpread) * ceil(n / kSpread) + w / kSpread instead: the warps resident at any time cover all
// destinations evenly (indices >= n fall out; spread_count(n) warps cover all rows).
constexpr int kSpread = 64;
__device__ __host__ __forceinline__ int64_t spread_count(int64_t n) { return (n + kSpread - 1) / kSpread * kSpread; }
__device__ __forceinline__ int64_t spread_row(int64_t w, int64_t n) {
  const int64_t per = (n + kSpread - 1) / kSpread;
  return (w % kSpread) * per + w / kSpread;
}

// One warp copies one row of K elements (16-byte pieces when `vec`), optionally scaled.
template <typename T>
__device__ __forceinline__ void copy_row(const T* __restrict__ src, T* __restrict__ dst, int K, bool vec, float sc,
                                         bool scaled, int lane) {
  if (vec) {
    constexpr int per = 16 / sizeof(T);
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const int n = K / per;
    // four loads in flight per lane before the first store: the stores may cross NVLink, and one 16-byte piece at a
    // time leaves the link idle between a load's return and the next one's issue
    for (int q0 = lane; q0 < n; q0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (q0 + 32 * u < n) v[u] = __ldg(s4 + q0 + 32 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (q0 + 32 * u >= n) break;
        if (scaled) {
          if constexpr (sizeof(T) == 4) {
            v[u].x = __float_as_uint(sc * __uint_as_float(v[u].x)); v[u].y = __float_as_uint(sc * __uint_as_float(v[u].y));
            v[u].z = __float_as_uint(sc * __uint_as_float(v[u].z)); v[u].w = __float_as_uint(sc * __uint_as_float(v[u].w));
          } else {
            uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float a = sc * __uint_as_float(w[i] << 16), b = sc * __uint_as_float(w[i] & 0xffff0000u);
              __nv_bfloat162 pk = __floats2bfloat162_rn(a, b);
              w[i] = *reinterpret_cast<uint32_t*>(&pk);
            }
            v[u] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        d4[q0 + 32 * u] = v[u];
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      if (!scaled) dst[k] = src[k];
      else if constexpr (sizeof(T) == 4) dst[k] = sc * src[k];
      else dst[k] = __float2bfloat16_rn(sc * __bfloat162float(src[k]));
    }
  }
}

// Sorted position i of this rank's slot list -> its row in the owner's receive buffer.
// The two exchange kernels run with 128 threads and at most 32 registers per thread, so that a block of them fits on
// an SM beside a 768-thread, 80-register CVMM block: rows of one micro-batch cross NVLink while the other
// micro-batch's projections run.
template <typename T>
__global__ void __launch_bounds__(128, 16) ep_put_kernel(const T* __restrict__ x, int64_t stride, int K, const int32_t* __restrict__ src_row,
                              int src_div, const float* __restrict__ row_scale, int64_t P,
                              const int32_t* __restrict__ sel_sorted, int El, const int32_t* __restrict__ plan,
                              const uint64_t* __restrict__ peer_ptrs, int G, int64_t peer_rows, int64_t x_rows, int vec,
                              int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t i = spread_row((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, P);
  if (i >= P) return;
  const int d = sel_sorted[i] / El;
  const int64_t sr = src_row[i];
  if (d < 0 || d >= G || sr < 0 || sr / src_div >= x_rows) {
    if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 51, static_cast<int>(i), static_cast<int>(sr));
    return;
  }
  const int64_t dst_row = static_cast<int64_t>(plan[2 + G + d]) + (i - plan[2 + d]);
  if (dst_row < 0 || dst_row >= peer_rows) {      // the row is dropped, and said so
    if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 52, static_cast<int>(i), static_cast<int>(dst_row));
    return;
  }
  T* dst = reinterpret_cast<T*>(peer_ptrs[d]) + dst_row * K;
  copy_row<T>(x + (sr / src_div) * stride, dst, K, vec != 0, row_scale ? row_scale[sr] : 1.f, row_scale != nullptr, lane);
}


// ep_put_kernel for fp32 gradient rows of the fp16 precision: the row (times its gate) is stored as fp16, scaled by the
// power of two of its own maximum, and the maximum goes to the same row of the destination's scale buffer.  Two passes
// over the source row (maximum, then conversion): the second one hits L1/L2.  Eight elements per lane and step, one
// 16-byte store each: a warp writes 512 contiguous bytes, as the plain copy does.
__global__ void __launch_bounds__(128, 16) ep_put_f16_kernel(const float* __restrict__ x, int64_t stride, int K,
                              const int32_t* __restrict__ src_row, int src_div, const float* __restrict__ row_scale, int64_t P,
                              const int32_t* __restrict__ sel_sorted, int El, const int32_t* __restrict__ plan,
                              const uint64_t* __restrict__ peer_ptrs, const uint64_t* __restrict__ scale_ptrs, int G,
                              int64_t peer_rows, int64_t x_rows, int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t i = spread_row((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, P);
  if (i >= P) return;
  const int d = sel_sorted[i] / El;
  const int64_t sr = src_row[i];
  if (d < 0 || d >= G || sr < 0 || sr / src_div >= x_rows) {
    if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 56, static_cast<int>(i), static_cast<int>(sr));
    return;
  }
  const int64_t dst_row = static_cast<int64_t>(plan[2 + G + d]) + (i - plan[2 + d]);
  if (dst_row < 0 || dst_row >= peer_rows) {      // the row is dropped, and said so
    if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 57, static_cast<int>(i), static_cast<int>(dst_row));
    return;
  }
  const float4* s4 = reinterpret_cast<const float4*>(x + (sr / src_div) * stride);
  const float sc = row_scale ? row_scale[sr] : 1.f;
  const int n8 = K / 8;
  float amax = 0.f;
  for (int q = lane; q < n8; q += 32) {
    const float4 a = __ldg(s4 + 2 * q), b = __ldg(s4 + 2 * q + 1);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax *= fabsf(sc);        // max|sc * v| (rounding of the product aside: a bound with a factor of two to spare)
  float inv;
  const float mul = sc * grad_pow2_scale(amax, inv);
  uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(peer_ptrs[d]) + dst_row * K);
  for (int q0 = lane; q0 < n8; q0 += 64) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (q0 + 32 * u < n8) { v[2 * u] = __ldg(s4 + 2 * (q0 + 32 * u)); v[2 * u + 1] = __ldg(s4 + 2 * (q0 + 32 * u) + 1); }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (q0 + 32 * u >= n8) break;
      const float4 a = v[2 * u], b = v[2 * u + 1];
      __half2 h0 = __floats2half2_rn(a.x * mul, a.y * mul), h1 = __floats2half2_rn(a.z * mul, a.w * mul);
      __half2 h2 = __floats2half2_rn(b.x * mul, b.y * mul), h3 = __floats2half2_rn(b.z * mul, b.w * mul);
      d4[q0 + 32 * u] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                                   *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    }
  }
  if (lane == 0) reinterpret_cast<float*>(scale_ptrs[d])[dst_row] = amax;
}

// Row r of this rank's receive-ordered buffer -> its place in the source rank's sorted slot list.
template <typename T>
__global__ void __launch_bounds__(128, 16) ep_put_back_kernel(const T* __restrict__ rows, int64_t stride, int K, const int32_t* __restrict__ plan,
                                   const uint64_t* __restrict__ peer_ptrs, int G, int64_t cap_rows, int64_t peer_rows,
                                   int vec, int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  if (plan[0] > cap_rows && blockIdx.x == 0 && threadIdx.x == 0)
    report(status, AMOE_ERR_INDEX_RANGE, 53, plan[0], static_cast<int>(cap_rows));
  const int64_t R = min(static_cast<int64_t>(plan[0]), cap_rows);
  const int32_t* recv_off = plan + 2 + 2 * G;
  const int32_t* back_off = plan + 2 + 3 * G;
  const int64_t n_spread = spread_count(R);
  for (int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < n_spread; w += warps) {
    const int64_t r = spread_row(w, R);
    if (r >= R) continue;
    int s = 0;
    for (int g = 1; g < G; ++g)
      if (recv_off[g] <= r) s = g;                    // last source whose block starts at or before r
    const int64_t dst_row = static_cast<int64_t>(back_off[s]) + (r - recv_off[s]);
    if (dst_row < 0 || dst_row >= peer_rows) {
      if (lane == 0) report(status, AMOE_ERR_INDEX_RANGE, 54, static_cast<int>(r), static_cast<int>(dst_row));
      continue;
    }
    copy_row<T>(rows + r * stride, reinterpret_cast<T*>(peer_ptrs[s]) + dst_row * K, K, vec != 0, 1.f, false, lane);
  }
}


// ---------------------------------------------------------------------------- small exchange + barrier in one launch
// Every rank hands a few bytes to every other rank and learns that all ranks have arrived: the count matrix of a step,
// a per-rank maximum, the column scales of the local experts - or nothing at all, when only the ordering of earlier
// peer stores matters.  One CTA: (1) this rank's payload is stored into slot [parity][rank] of every rank's slot
// buffer; (2) thread p raises this rank's flag in rank p's flag array to the new epoch (release, system scope) and waits
// until rank p's flag in the own array has reached it (acquire, system scope); (3) the G payloads are copied out of the
// own slot buffer.  Epochs only grow (a device counter per rank, advanced by this kernel, so a captured graph replays
// correctly); payload slots alternate with the epoch's parity: a rank can only be one exchange ahead of the slowest
// reader, never two.  Every wait is bounded: after `spin_limit` polls the kernel records AMOE_ERR_WAIT_LIMIT and returns.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(1024) ep_share_kernel(const uint32_t* __restrict__ payload, int words,
                                                       const uint64_t* __restrict__ slot_ptrs, int64_t slot_words,
                                                       const uint64_t* __restrict__ flag_ptrs, uint32_t* __restrict__ epoch_ctr,
                                                       int me, int G, uint32_t* __restrict__ out, long long spin_limit,
                                                       int32_t* __restrict__ status) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_gave_up;
  // an earlier exchange that gave up is latched in the status word: do not wait the limit out again on every call
  if (threadIdx.x == 0) { s_epoch = *epoch_ctr + 1u; s_gave_up = (status != nullptr && status[0] == AMOE_ERR_WAIT_LIMIT) ? 1 : 0; }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int64_t par = epoch & 1u;
  // (16-byte pieces when everything is aligned for them: the larger payloads are a few tens of KB)
  const bool vec = (words % 4 == 0) && (slot_words % 4 == 0) && ((reinterpret_cast<uintptr_t>(payload) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  for (int p = 0; p < G; ++p) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(slot_ptrs[p]) + (par * G + me) * slot_words;
    if (vec) {
      for (int w = threadIdx.x; w < words / 4; w += blockDim.x)
        reinterpret_cast<uint4*>(dst)[w] = __ldg(reinterpret_cast<const uint4*>(payload) + w);
    } else {
      for (int w = threadIdx.x; w < words; w += blockDim.x) dst[w] = payload[w];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < G) {
    const int p = threadIdx.x;
    st_release_sys(reinterpret_cast<uint32_t*>(flag_ptrs[p]) + me, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flag_ptrs[me]) + p;
    long long polls = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (s_gave_up || ++polls > spin_limit) {
        s_gave_up = 1;
        report(status, AMOE_ERR_WAIT_LIMIT, 55, p, static_cast<int>(epoch));
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
  if (out != nullptr && !s_gave_up) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(slot_ptrs[me]) + par * G * slot_words;
    for (int g = 0; g < G; ++g) {
      if (vec) {
        // (plain loads: the other ranks wrote these slots during this kernel)
        for (int w = threadIdx.x; w < words / 4; w += blockDim.x)
          reinterpret_cast<uint4*>(out + static_cast<int64_t>(g) * words)[w] = reinterpret_cast<const uint4*>(src + g * slot_words)[w];
      } else {
        for (int w = threadIdx.x; w < words; w += blockDim.x) out[static_cast<int64_t>(g) * words + w] = src[g * slot_words + w];
      }
    }
  }
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace amoe

using namespace amoe;

extern "C" {

int64_t amoe_ep_plan_ints(int32_t G, int32_t El) { return G > 0 && El > 0 ? plan_ints(G, El) : 0; }

int amoe_ep_plan(const int32_t* gathered, int32_t rank, int32_t G, int32_t El, int32_t* plan, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(gathered && plan, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(G > 0 && G <= kEpMaxRanks && El > 0 && rank >= 0 && rank < G && G * El <= kEpMaxBlocksDev, AMOE_ERR_BAD_SHAPE);
  ep_plan_kernel<<<1, 256, 0, stream>>>(gathered, rank, G, El, plan);
  AMOE_LAUNCH_CHECK("ep_plan");
  return AMOE_OK;
}

int amoe_ep_local_plan_dev(const int32_t* plan, int32_t G, int32_t El, int64_t cap_rows, int32_t* local_order,
                           int32_t* local_offsets, int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(plan && local_order && local_offsets, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(G > 0 && El > 0 && G * El <= kEpMaxBlocksDev && cap_rows > 0 && cap_rows < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  int64_t blocks = (cap_rows + 255) / 256;
  if (blocks > 592) blocks = 592;
  ep_local_plan_dev_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(plan, G, El, static_cast<int>(cap_rows), local_order,
                                                                             local_offsets, dev_status);
  AMOE_LAUNCH_CHECK("ep_local_plan_dev");
  return AMOE_OK;
}

int amoe_ep_put(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows, const int32_t* src_row,
                int32_t src_div, const float* row_scale, int64_t P, const int32_t* sel_sorted, int32_t El,
                const int32_t* plan, const uint64_t* peer_ptrs, int32_t G, int64_t peer_rows, int32_t* dev_status,
                amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && src_row && sel_sorted && plan && peer_ptrs, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && K > 0 && El > 0 && G > 0 && G <= kEpMaxRanks && src_div >= 1 && peer_rows > 0 && x_rows > 0, AMOE_ERR_BAD_SHAPE);
  const int esz = dtype == AMOE_F32 ? 4 : 2;
  const int vec = al16(x) && (stride * esz) % 16 == 0 && (static_cast<int64_t>(K) * esz) % 16 == 0;   // peer bases are page aligned
  const unsigned blocks = static_cast<unsigned>((spread_count(P) * 32 + 127) / 128);
  if (dtype == AMOE_F32)
    ep_put_kernel<float><<<blocks, 128, 0, stream>>>(reinterpret_cast<const float*>(x), stride, K, src_row, src_div, row_scale, P,
                                                     sel_sorted, El, plan, peer_ptrs, G, peer_rows, x_rows, vec, dev_status);
  else if (dtype == AMOE_BF16)
    ep_put_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), stride, K, src_row, src_div,
                                                             row_scale, P, sel_sorted, El, plan, peer_ptrs, G, peer_rows, x_rows,
                                                             vec, dev_status);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("ep_put");
  return AMOE_OK;
}

int amoe_ep_put_f16(const float* x, int64_t stride, int32_t K, int64_t x_rows, const int32_t* src_row, int32_t src_div,
                    const float* row_scale, int64_t P, const int32_t* sel_sorted, int32_t El, const int32_t* plan,
                    const uint64_t* peer_ptrs, const uint64_t* scale_ptrs, int32_t G, int64_t peer_rows,
                    int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(x && src_row && sel_sorted && plan && peer_ptrs && scale_ptrs, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(P > 0 && K > 0 && K % 8 == 0 && El > 0 && G > 0 && G <= kEpMaxRanks && src_div >= 1 && peer_rows > 0 && x_rows > 0,
               AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(al16(x) && (stride * 4) % 16 == 0, AMOE_ERR_BAD_SHAPE);      // peer bases are page aligned
  const unsigned blocks = static_cast<unsigned>((spread_count(P) * 32 + 127) / 128);
  ep_put_f16_kernel<<<blocks, 128, 0, stream>>>(x, stride, K, src_row, src_div, row_scale, P, sel_sorted, El, plan, peer_ptrs,
                                                scale_ptrs, G, peer_rows, x_rows, dev_status);
  AMOE_LAUNCH_CHECK("ep_put_f16");
  return AMOE_OK;
}

int amoe_ep_put_back(const void* rows, int32_t dtype, int64_t stride, int32_t K, const int32_t* plan,
                     const uint64_t* peer_ptrs, int32_t G, int64_t cap_rows, int64_t peer_rows, int32_t* dev_status,
                     amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(rows && plan && peer_ptrs, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(K > 0 && G > 0 && G <= kEpMaxRanks && cap_rows > 0 && peer_rows > 0, AMOE_ERR_BAD_SHAPE);
  const int esz = dtype == AMOE_F32 ? 4 : 2;
  const int vec = al16(rows) && (stride * esz) % 16 == 0 && (static_cast<int64_t>(K) * esz) % 16 == 0;
  int64_t blocks = (cap_rows * 32 + 127) / 128;
  const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  if (dtype == AMOE_F32)
    ep_put_back_kernel<float><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(reinterpret_cast<const float*>(rows), stride, K, plan,
                                                                                 peer_ptrs, G, cap_rows, peer_rows, vec, dev_status);
  else if (dtype == AMOE_BF16)
    ep_put_back_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(rows), stride, K, plan, peer_ptrs, G, cap_rows, peer_rows, vec, dev_status);
  else
    return AMOE_ERR_BAD_DTYPE;
  AMOE_LAUNCH_CHECK("ep_put_back");
  return AMOE_OK;
}

int amoe_ep_share(const void* payload, int64_t nbytes, const uint64_t* slot_ptrs, int64_t slot_bytes,
                  const uint64_t* flag_ptrs, uint32_t* epoch, int32_t rank, int32_t G, void* gathered,
                  int64_t spin_limit, int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(slot_ptrs && flag_ptrs && epoch, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(nbytes == 0 || payload != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(G > 0 && G <= kEpMaxRanks && rank >= 0 && rank < G && nbytes >= 0 && nbytes % 4 == 0 && slot_bytes % 4 == 0 &&
               nbytes <= slot_bytes && spin_limit > 0, AMOE_ERR_BAD_SHAPE);
  ep_share_kernel<<<1, nbytes > 4096 ? 1024 : 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(payload), static_cast<int>(nbytes / 4), slot_ptrs,
                                         slot_bytes / 4, flag_ptrs, epoch, rank, G, reinterpret_cast<uint32_t*>(gathered),
                                         spin_limit, dev_status);
  AMOE_LAUNCH_CHECK("ep_share");
  return AMOE_OK;
}

}  // extern "C"
