// Row-owner epilogue shared by the CUDA-core and the tcgen05 CVMM kernels.
//
// One thread owns one output row (one sorted position) - or, in the tcgen05 kernel, an interleaved
// share of that row's 16-column chunks - and walks its columns four at a time, so that every
// per-row reduction (the input-range gradient) is a fixed-order sum.
#pragma once
#include "common.cuh"

namespace amoe {

struct EpiParams {
  int is_dx;            // 0: forward epilogue, 1: input-gradient epilogue
  int n_out;            // output columns
  int vec4;             // n_out % 4 == 0 and every per-column / per-row array is 16-byte aligned
  // forward
  const float* noise; float noise_std; uint64_t seed; uint32_t offset; const long long* step_dev;
  uint32_t pkeys[20];   // Philox round keys of `seed`
  const float* col_scale;      // [E, n_out]
  const float* col_inv_scale;  // [E, n_out], needed by the ADC
  AdcParams adc;
  const float* a_absmax; const float* ir;  // by source row / by sorted position (by expert if ir_by_expert)
  int ir_by_expert;
  int out_relu;         // forward: clamp the result at zero
  int x_ref_relu;       // input gradient: also zero the result where x_ref <= 0
  const int32_t* a_row; const int32_t* dst_row; int a_div;
  int64_t a_rows, dst_rows;
  float acc_mul;        // multiplies the raw accumulator (the DAC resolution when A holds integer codes)
  void* out; int out_dtype; int64_t out_stride; int8_t* out_codes;
  float* out_row_scale; int32_t* out_row_expert;
  // input gradient
  const void* x_ref; int x_ref_dtype; int64_t x_ref_stride; int64_t x_ref_rows; const int32_t* x_ref_row;
  const float* row_scale; float* ir_grad; int relative; float grad_scale;
  unsigned long long* keep_count;
  // input gradient, optional: the result rows once more as bf16 hi (+ lo) terms, by padded tile row
  __nv_bfloat16* out_cache_hi; __nv_bfloat16* out_cache_lo; int64_t out_cache_stride;
  // forward, optional: the result as the next projection's operands (see amoe_cvmm_args)
  const float* next_ir; float next_res; __nv_bfloat16* next_codes; const float* out_cache_scale;
  int32_t* status;
};

struct RowCtx {
  int valid;       // row takes part (inside the expert's run and all indices in range)
  int e;
  int64_t dst;
  float ir;
  float absmax;
  float rs;
  int64_t xrow;
  float dir_acc;
  unsigned keep;
  uint32_t noise_offset;   // Philox offset in effect (argument + 8 * device step counter)
  int64_t pad_row;         // tile index * 128 + row in tile (row of the operand caches)
  float next_ir, next_rcp; // input range of the next projection for this row's expert and its reciprocal
  float out_cache_sc;      // out_cache_scale of this row (1 when absent), fetched once per tile
};

__device__ __forceinline__ RowCtx epi_row_begin(const EpiParams& p, int64_t i, int e, bool in_range) {
  RowCtx c;
  c.valid = in_range;
  c.e = e;
  c.dst = 0; c.ir = 1.f; c.absmax = 1.f; c.rs = 1.f; c.xrow = 0; c.dir_acc = 0.f; c.keep = 0;
  c.noise_offset = p.offset;
  c.pad_row = 0;
  c.next_ir = 1.f; c.next_rcp = 1.f; c.out_cache_sc = 1.f;
  if (!p.is_dx && p.next_ir) { c.next_ir = p.next_ir[e]; c.next_rcp = __frcp_rn(c.next_ir); }
  if (p.noise_std > 0.f && p.step_dev) c.noise_offset += static_cast<uint32_t>(*p.step_dev) * 8u;
  if (!in_range) return c;
  c.dst = p.dst_row[i];
  if (c.dst < 0 || c.dst >= p.dst_rows) {
    report(p.status, AMOE_ERR_INDEX_RANGE, 10, static_cast<int>(i), static_cast<int>(c.dst));
    c.valid = 0;
    return c;
  }
  if (p.ir) c.ir = p.ir[p.ir_by_expert ? e : i];
  if (!p.is_dx) {
    if (p.a_absmax) {
      int64_t r = p.a_row[i] / p.a_div;
      if (r >= 0 && r < p.a_rows) c.absmax = p.a_absmax[r];
    }
  } else {
    if (p.row_scale) c.rs = p.row_scale[c.dst];
    if (p.x_ref) {
      c.xrow = p.x_ref_row[i];
      if (c.xrow < 0 || c.xrow >= p.x_ref_rows) {
        report(p.status, AMOE_ERR_INDEX_RANGE, 11, static_cast<int>(i), static_cast<int>(c.xrow));
        c.valid = 0;
      }
    }
  }
  return c;
}

__device__ __forceinline__ void load4(const float* base, int64_t idx, int n0, int n_out, bool vec, float o[4], float fill) {
  if (vec) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(base + idx));
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = (n0 + j < n_out) ? base[idx + j] : fill;
  }
}

// Four consecutive columns n0..n0+3 (n0 % 4 == 0) of the row; v = raw accumulators.
__device__ __forceinline__ void epi_quad(const EpiParams& p, RowCtx& c, int n0, const float v[4]) {
  if (!c.valid || n0 >= p.n_out) return;
  const bool vec = p.vec4 != 0;      // implies n0 + 3 < n_out
  float o[4];
  float code[4] = {0.f, 0.f, 0.f, 0.f};
  if (!p.is_dx) {
    const int64_t cidx = static_cast<int64_t>(c.e) * p.n_out + n0;
    float s[4] = {1.f, 1.f, 1.f, 1.f}, is[4] = {1.f, 1.f, 1.f, 1.f}, nz[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.col_scale) load4(p.col_scale, cidx, n0, p.n_out, vec, s, 1.f);
    if (p.adc.on) load4(p.col_inv_scale, cidx, n0, p.n_out, vec, is, 0.f);
    if (p.noise) load4(p.noise, c.dst * p.n_out + n0, n0, p.n_out, vec, nz, 0.f);
    if (p.noise_std > 0.f) {
      const float4 zz = philox_normal8_half(p.seed, c.noise_offset, kStreamOutNoise, static_cast<uint32_t>(c.dst),
                                            static_cast<uint32_t>(n0 >> 2));
      nz[0] += (p.noise_std * s[0]) * zz.x;
      nz[1] += (p.noise_std * s[1]) * zz.y;
      nz[2] += (p.noise_std * s[2]) * zz.z;
      nz[3] += (p.noise_std * s[3]) * zz.w;
    }
    const float post = c.absmax * c.ir;   // both 1 when absent; only one of the two is used in practice
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float acc = v[j] * p.acc_mul + nz[j];
      if (p.adc.on) acc = adc_apply(acc, s[j], is[j], p.adc, code[j]);
      if (p.a_absmax && p.ir) acc = (acc * c.absmax) * c.ir;
      else acc *= post;
      if (p.out_relu) acc = fmaxf(acc, 0.f);
      o[j] = acc;
    }
  } else {
    float xr[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.x_ref) {
      const int64_t xi = c.xrow * p.x_ref_stride + n0;
      if (vec && p.x_ref_dtype == AMOE_F32) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x_ref) + xi));
        xr[0] = t.x; xr[1] = t.y; xr[2] = t.z; xr[3] = t.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n0 + j < p.n_out) xr[j] = load_elem(p.x_ref, p.x_ref_dtype, xi + j);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gs = v[j] * c.rs;
      if (p.x_ref && n0 + j < p.n_out) {
        if (p.ir) {
          const bool up = xr[j] >= c.ir, low = xr[j] <= -c.ir, keep = fabsf(xr[j]) < c.ir;
          if (up) c.dir_acc += fminf(gs, 0.f);
          if (low) c.dir_acc -= fmaxf(gs, 0.f);
          c.keep += keep ? 1u : 0u;
          gs = keep ? gs : 0.f;
        }
        if (p.x_ref_relu && !(xr[j] > 0.f)) gs = 0.f;
      }
      o[j] = gs;
    }
  }
  const int64_t base = c.dst * p.out_stride + n0;
  if (p.out == nullptr) {
    // codes only
  } else if (vec && p.out_dtype == AMOE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + base) = make_float4(o[0], o[1], o[2], o[3]);
  } else if (vec) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + base) = pk;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n0 + j < p.n_out) store_elem(p.out, p.out_dtype, base + j, o[j]);
  }
  if (p.out_codes) {
    if (vec) {
      const uint32_t pk = (static_cast<uint32_t>(static_cast<int>(code[0])) & 0xffu) |
                          ((static_cast<uint32_t>(static_cast<int>(code[1])) & 0xffu) << 8) |
                          ((static_cast<uint32_t>(static_cast<int>(code[2])) & 0xffu) << 16) |
                          ((static_cast<uint32_t>(static_cast<int>(code[3])) & 0xffu) << 24);
      *reinterpret_cast<uint32_t*>(p.out_codes + c.dst * p.n_out + n0) = pk;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < p.n_out) p.out_codes[c.dst * p.n_out + n0 + j] = static_cast<int8_t>(code[j]);
    }
  }
}

// Per-row side outputs of the forward epilogue (written once per row by its owner).
__device__ __forceinline__ void epi_row_side_outputs(const EpiParams& p, const RowCtx& c) {
  if (p.is_dx || !c.valid) return;
  if (p.out_row_scale) p.out_row_scale[c.dst] = c.absmax * c.ir;
  if (p.out_row_expert) p.out_row_expert[c.dst] = c.e;
}

// After the last column: per-row results of the input-gradient epilogue (dir_acc already complete).
__device__ __forceinline__ void epi_row_end(const EpiParams& p, RowCtx& c, int64_t i) {
  if (!p.is_dx || !c.valid) return;
  if (p.ir_grad) {
    float d = c.dir_acc;
    if (p.relative) d = (d * c.ir) * p.grad_scale;
    p.ir_grad[i] = d;
  }
}

}  // namespace amoe
