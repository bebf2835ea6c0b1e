// Gate select (sigmoid + top-k) and the stable expert-contiguous slot sort.
//
// Five small kernels, no host synchronisation, no atomics on the data path, so the slot order is a
// pure function of the logits:
//   topk_kernel      one warp per token: k rounds of warp arg-max over the E gate values
//   chunk_hist       one warp per chunk of kChunk flat slots: per-expert counts of the chunk
//   chunk_scan       one warp per expert: exclusive prefix of its counts over the chunks
//   offsets_kernel   one CTA: exclusive scan of the expert totals -> expert_offsets
//   scatter_kernel   one warp per chunk: stable rank inside the chunk via match.any
#include "common.cuh"

namespace amoe {
namespace {

constexpr int kChunk = 256;    // flat slots per warp in the sort
constexpr int kMaxE = 1024;
constexpr int kMaxK = 32;

// kPer = experts per lane (E <= 32 * kPer): the arg-max loops are unrolled over exactly that many.
template <int kPer>
__global__ void topk_kernel(const float* __restrict__ logits, int64_t T, int E, int k, int apply_sigmoid,
                            int32_t* __restrict__ raw_sel, float* __restrict__ gate) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  // each lane holds experts lane, lane+32, ...
  float v[kPer];
  const float* row = logits + t * E;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    int e = lane + 32 * i;
    float x = -INFINITY;
    if (e < E) {
      x = row[e];
      if (apply_sigmoid) x = 1.0f / (1.0f + expf(-x));
    }
    v[i] = x;
  }
  constexpr int per = kPer;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      if (i < per) {
        int e = lane + 32 * i;
        // NaN never wins; ties go to the lower expert id
        if (e < E && (v[i] > best || (v[i] == best && e < best_e))) {
          best = v[i];
          best_e = e;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if (best_e == 0x7fffffff) best_e = j;  // all-NaN row: keep indices in range
    if (lane == 0) {
      raw_sel[t * k + j] = best_e;
      gate[t * k + j] = best;
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (i == (best_e >> 5)) v[i] = -INFINITY;
    }
  }
}

__global__ void chunk_hist_kernel(const int32_t* __restrict__ raw_sel, int64_t P, int E,
                                  int32_t* __restrict__ hist /*[nchunks,E]*/) {
  extern __shared__ int32_t cnt[];  // [warps_per_block][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  int32_t* my = cnt + warp * E;
  for (int e = lane; e < E; e += 32) my[e] = 0;
  __syncwarp();
  const int64_t s0 = chunk * kChunk;
  if (s0 < P) {
    for (int64_t s = s0 + lane; s < s0 + kChunk; s += 32) {
      bool ok = s < P;
      int e = ok ? raw_sel[s] : -1;
      ok = ok && e >= 0 && e < E;
      unsigned m = __match_any_sync(0xffffffffu, ok ? e : -1);
      if (ok && (__ffs(m) - 1) == lane) my[e] += __popc(m);
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) hist[chunk * E + e] = my[e];
  }
}

// Per expert (one warp each): exclusive prefix of its counts over the chunks, in place, and its total.
__global__ void chunk_scan_kernel(int32_t* __restrict__ hist, int64_t nchunks, int E, int32_t* __restrict__ total) {
  const int lane = threadIdx.x & 31;
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (e >= E) return;
  int32_t carry = 0;
  for (int64_t c0 = 0; c0 < nchunks; c0 += 32) {
    const int64_t c = c0 + lane;
    const int32_t h = c < nchunks ? hist[c * E + e] : 0;
    int32_t incl = h;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (c < nchunks) hist[c * E + e] = carry + incl - h;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) total[e] = carry;
}

// offsets[E+1] = exclusive scan of the per-expert totals (one CTA; E <= 1024).
__global__ void offsets_kernel(const int32_t* __restrict__ total, int E, int32_t* __restrict__ offsets) {
  __shared__ int32_t warp_sum[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = threadIdx.x;
  const int32_t h = e < E ? total[e] : 0;
  int32_t incl = h;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t w = warp_sum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += up;
    }
    warp_sum[lane] = w;
  }
  __syncthreads();
  const int32_t base = warp > 0 ? warp_sum[warp - 1] : 0;
  if (e < E) offsets[e] = base + incl - h;
  if (e == E - 1) offsets[E] = base + incl;
}

__global__ void scatter_kernel(const int32_t* __restrict__ raw_sel, int64_t P, int E, int k,
                               const int32_t* __restrict__ base /*[nchunks,E] prefix inside the expert*/,
                               const int32_t* __restrict__ offsets, int32_t* __restrict__ sel_sorted,
                               int32_t* __restrict__ token_index, int32_t* __restrict__ slot_index) {
  extern __shared__ int32_t cnt[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  const int64_t s0 = chunk * kChunk;
  if (s0 >= P) return;
  int32_t* my = cnt + warp * E;
  for (int e = lane; e < E; e += 32) my[e] = offsets[e] + base[chunk * E + e];
  __syncwarp();
  for (int64_t s = s0 + lane; s < s0 + kChunk; s += 32) {
    bool ok = s < P;
    int e = ok ? raw_sel[s] : -1;
    ok = ok && e >= 0 && e < E;
    unsigned m = __match_any_sync(0xffffffffu, ok ? e : -1);
    int pos = 0;
    if (ok) pos = my[e] + __popc(m & ((1u << lane) - 1u));
    __syncwarp();
    if (ok && (__ffs(m) - 1) == lane) my[e] += __popc(m);
    __syncwarp();
    if (ok) {
      sel_sorted[pos] = e;
      slot_index[pos] = static_cast<int32_t>(s);
      token_index[pos] = static_cast<int32_t>(s / k);
    }
  }
}

// Scan + offsets + scatter in one kernel for moderate sizes: every warp (one chunk) sums the histogram columns itself
// (its own exclusive prefix over the earlier chunks and the experts' totals), which is nchunks * E loads per warp from
// a table that sits in L2, instead of waiting for two more kernels.  Same positions as the three-kernel path.
__global__ void scan_scatter_kernel(const int32_t* __restrict__ raw_sel, int64_t P, int E, int k,
                                    const int32_t* __restrict__ hist /*[nchunks,E] counts*/, int64_t nchunks,
                                    int32_t* __restrict__ offsets, int32_t* __restrict__ sel_sorted,
                                    int32_t* __restrict__ token_index, int32_t* __restrict__ slot_index) {
  extern __shared__ int32_t cnt[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  const int64_t s0 = chunk * kChunk;
  if (s0 >= P) return;
  int32_t* my = cnt + warp * E;
  int32_t carry = 0;                                   // total of all experts below the current group of 32
  // with fewer than 32 experts the lanes also split the chunk range: lane = part * ew + expert
  int ew = 32;
  while (ew > 1 && (ew >> 1) >= E) ew >>= 1;           // experts per group, rounded up to a power of two (<= 32)
  const int parts = 32 / ew;
  for (int e0 = 0; e0 < E; e0 += ew) {
    const int e = e0 + (lane & (ew - 1));
    const int part = lane / ew;
    const int64_t c_lo = nchunks * part / parts, c_hi = nchunks * (part + 1) / parts;
    int32_t tot = 0, pre = 0;
    if (e < E) {
#pragma unroll 8
      for (int64_t c = c_lo; c < c_hi; ++c) {
        const int32_t h = hist[c * E + e];
        tot += h;
        if (c < chunk) pre += h;
      }
    }
    for (int o = ew; o < 32; o <<= 1) {                // sum over the parts: afterwards every lane of an expert has both
      tot += __shfl_xor_sync(0xffffffffu, tot, o);
      pre += __shfl_xor_sync(0xffffffffu, pre, o);
    }
    int32_t incl = (lane < ew) ? tot : 0;              // scan over the experts in the first ew lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const int32_t start = carry + incl - tot;          // first sorted position of expert e (valid for lane < ew)
    if (lane < ew && e < E) {
      my[e] = start + pre;
      if (chunk == 0) offsets[e] = start;
    }
    carry += __shfl_sync(0xffffffffu, incl, ew - 1);
  }
  if (chunk == 0 && lane == 0) offsets[E] = carry;
  __syncwarp();
  for (int64_t s = s0 + lane; s < s0 + kChunk; s += 32) {
    bool ok = s < P;
    int e = ok ? raw_sel[s] : -1;
    ok = ok && e >= 0 && e < E;
    unsigned m = __match_any_sync(0xffffffffu, ok ? e : -1);
    int pos = 0;
    if (ok) pos = my[e] + __popc(m & ((1u << lane) - 1u));
    __syncwarp();
    if (ok && (__ffs(m) - 1) == lane) my[e] += __popc(m);
    __syncwarp();
    if (ok) {
      sel_sorted[pos] = e;
      slot_index[pos] = static_cast<int32_t>(s);
      token_index[pos] = static_cast<int32_t>(s / k);
    }
  }
}

__global__ void offsets_from_sorted_kernel(const int32_t* __restrict__ sel, int64_t P, int E,
                                           int32_t* __restrict__ offsets, int32_t* status) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i > P) return;
  int prev = i == 0 ? -1 : sel[i - 1];
  int cur = i == P ? E : sel[i];
  if (i < P && (cur < 0 || cur >= E)) {
    report(status, AMOE_ERR_INDEX_RANGE, 1, static_cast<int>(i), cur);
    cur = cur < 0 ? 0 : E - 1;
  }
  if (prev < -1) prev = -1;
  if (prev >= E) prev = E - 1;
  if (cur < prev) {  // not sorted
    report(status, AMOE_ERR_INDEX_RANGE, 2, static_cast<int>(i), cur);
    return;
  }
  for (int e = prev + 1; e <= cur; ++e) offsets[e] = static_cast<int32_t>(i);
}

// dlogits[t,e] = dgate[t,j] * dsigmoid for the slot j of token t that picked expert e, else 0.
__global__ void gate_backward_kernel(const float* __restrict__ dgate, const float* __restrict__ gate,
                                     const int32_t* __restrict__ raw_sel, int64_t T, int E, int k, int apply_sigmoid,
                                     float* __restrict__ dlogits) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= T * E) return;
  const int64_t t = i / E;
  const int e = static_cast<int>(i - t * E);
  float v = 0.f;
  for (int j = 0; j < k; ++j) {
    if (raw_sel[t * k + j] == e) {
      const float g = gate[t * k + j];
      v = apply_sigmoid ? (dgate[t * k + j] * (1.f - g)) * g : dgate[t * k + j];
    }
  }
  dlogits[i] = v;
}

}  // namespace
}  // namespace amoe

using namespace amoe;

static int sort_slots(const int32_t* raw_sel, int64_t T, int32_t E, int32_t k, int32_t* sel_sorted, int32_t* token_index,
                      int32_t* slot_index, int32_t* expert_offsets, void* workspace, cudaStream_t stream) {
  const int64_t P = T * k;
  const int64_t nchunks = (P + kChunk - 1) / kChunk;
  int32_t* hist = reinterpret_cast<int32_t*>(workspace);
  // warps per block limited by shared memory: E ints per warp
  int wpb = 8;
  while (wpb > 1 && static_cast<size_t>(wpb) * E * sizeof(int32_t) > 32 * 1024) wpb >>= 1;
  const unsigned blocks = static_cast<unsigned>((nchunks + wpb - 1) / wpb);
  const size_t smem = static_cast<size_t>(wpb) * E * sizeof(int32_t);
  chunk_hist_kernel<<<blocks, wpb * 32, smem, stream>>>(raw_sel, P, E, hist);
  AMOE_LAUNCH_CHECK("chunk_hist");
  if (nchunks * E <= 8192) {      // each warp reads the whole table: keep that to 32 KiB
    scan_scatter_kernel<<<blocks, wpb * 32, smem, stream>>>(raw_sel, P, E, k, hist, nchunks, expert_offsets, sel_sorted,
                                                           token_index, slot_index);
    AMOE_LAUNCH_CHECK("scan_scatter");
    return AMOE_OK;
  }
  int32_t* total = hist + nchunks * E;
  chunk_scan_kernel<<<(E * 32 + 255) / 256, 256, 0, stream>>>(hist, nchunks, E, total);
  AMOE_LAUNCH_CHECK("chunk_scan");
  offsets_kernel<<<1, 1024, 0, stream>>>(total, E, expert_offsets);
  AMOE_LAUNCH_CHECK("offsets");
  scatter_kernel<<<blocks, wpb * 32, smem, stream>>>(raw_sel, P, E, k, hist, expert_offsets, sel_sorted, token_index,
                                                     slot_index);
  AMOE_LAUNCH_CHECK("scatter");
  return AMOE_OK;
}

extern "C" {

size_t amoe_select_sort_workspace_bytes(int64_t T, int32_t E, int32_t k) {
  if (T <= 0 || E <= 0 || k <= 0) return 0;
  int64_t P = T * k;
  int64_t nchunks = (P + kChunk - 1) / kChunk;
  return (static_cast<size_t>(nchunks) * E + E) * sizeof(int32_t);
}

int amoe_select_sort(const float* logits, int64_t T, int32_t E, int32_t k, int32_t apply_sigmoid, int32_t* raw_sel,
                     float* gate, int32_t* sel_sorted, int32_t* token_index, int32_t* slot_index,
                     int32_t* expert_offsets, void* workspace, size_t workspace_bytes, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(T > 0 && E > 0 && k > 0 && E <= kMaxE && k <= kMaxK && k <= E, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(T * k < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(logits && raw_sel && gate && sel_sorted && token_index && slot_index && expert_offsets,
               AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(workspace && workspace_bytes >= amoe_select_sort_workspace_bytes(T, E, k), AMOE_ERR_WORKSPACE);
  {
    const int threads = 256;
    const int64_t blocks = (T * 32 + threads - 1) / threads;
    const unsigned nb = static_cast<unsigned>(blocks);
    if (E <= 32) topk_kernel<1><<<nb, threads, 0, stream>>>(logits, T, E, k, apply_sigmoid, raw_sel, gate);
    else if (E <= 64) topk_kernel<2><<<nb, threads, 0, stream>>>(logits, T, E, k, apply_sigmoid, raw_sel, gate);
    else if (E <= 128) topk_kernel<4><<<nb, threads, 0, stream>>>(logits, T, E, k, apply_sigmoid, raw_sel, gate);
    else if (E <= 256) topk_kernel<8><<<nb, threads, 0, stream>>>(logits, T, E, k, apply_sigmoid, raw_sel, gate);
    else topk_kernel<kMaxE / 32><<<nb, threads, 0, stream>>>(logits, T, E, k, apply_sigmoid, raw_sel, gate);
    AMOE_LAUNCH_CHECK("topk");
  }
  return sort_slots(raw_sel, T, E, k, sel_sorted, token_index, slot_index, expert_offsets, workspace, stream);
}

int amoe_sort_slots(const int32_t* raw_sel, int64_t T, int32_t E, int32_t k, int32_t* sel_sorted, int32_t* token_index,
                    int32_t* slot_index, int32_t* expert_offsets, void* workspace, size_t workspace_bytes,
                    amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(T > 0 && E > 0 && k > 0 && E <= kMaxE && k <= kMaxK && k <= E, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(T * k < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(raw_sel && sel_sorted && token_index && slot_index && expert_offsets, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(workspace && workspace_bytes >= amoe_select_sort_workspace_bytes(T, E, k), AMOE_ERR_WORKSPACE);
  return sort_slots(raw_sel, T, E, k, sel_sorted, token_index, slot_index, expert_offsets, workspace, stream);
}

int amoe_gate_backward(const float* dgate, const float* gate, const int32_t* raw_sel, int64_t T, int32_t E, int32_t k,
                       int32_t apply_sigmoid, float* dlogits, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(T > 0 && E > 0 && k > 0 && k <= E, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(dgate && gate && raw_sel && dlogits, AMOE_ERR_NULL_POINTER);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((T * E + threads - 1) / threads);
  gate_backward_kernel<<<blocks, threads, 0, stream>>>(dgate, gate, raw_sel, T, E, k, apply_sigmoid, dlogits);
  AMOE_LAUNCH_CHECK("gate_backward");
  return AMOE_OK;
}

int amoe_expert_offsets(const int32_t* sel_sorted, int64_t P, int32_t E, int32_t* expert_offsets,
                        int32_t* dev_status, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(P > 0 && E > 0 && P < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(sel_sorted && expert_offsets, AMOE_ERR_NULL_POINTER);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((P + 1 + threads - 1) / threads);
  offsets_from_sorted_kernel<<<blocks, threads, 0, stream>>>(sel_sorted, P, E, expert_offsets, dev_status);
  AMOE_LAUNCH_CHECK("offsets_from_sorted");
  return AMOE_OK;
}

}  // extern "C"
