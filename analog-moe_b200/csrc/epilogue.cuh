// Row-owner epilogue shared by the CUDA-core and the tcgen05 CVMM kernels.
//
// One thread owns one output row (one sorted position) and walks its columns four at a time, so
// that every per-row reduction (the input-range gradient) is a thread-local, order-fixed sum.
#pragma once
#include "common.cuh"

namespace amoe {

struct EpiParams {
  int is_dx;            // 0: forward epilogue, 1: input-gradient epilogue
  int n_out;            // output columns
  // forward
  const float* noise; float noise_std; uint64_t seed; uint32_t offset;
  const float* col_scale;  // [E, n_out]
  AdcParams adc;
  const float* a_absmax; const float* ir;  // by source row / by sorted position
  const int32_t* a_row; const int32_t* dst_row; int a_div;
  int64_t a_rows, dst_rows;
  float acc_mul;        // multiplies the raw accumulator (the DAC resolution when A holds integer codes)
  void* out; int out_dtype; int64_t out_stride; int8_t* out_codes;
  // input gradient
  const void* x_ref; int x_ref_dtype; int64_t x_ref_stride; int64_t x_ref_rows; const int32_t* x_ref_row;
  const float* row_scale; float* ir_grad; int relative; float grad_scale;
  unsigned long long* keep_count;
  int32_t* status;
};

struct RowCtx {
  int valid;       // row takes part (inside the expert's run and all indices in range)
  int e;
  int64_t dst;
  float ir, post;  // input range of the row, and absmax*... multiplier applied last
  float absmax;
  float rs;
  int64_t xrow;
  float dir_acc;
  unsigned keep;
};

__device__ __forceinline__ RowCtx epi_row_begin(const EpiParams& p, int64_t i, int e, bool in_range) {
  RowCtx c;
  c.valid = in_range;
  c.e = e;
  c.dst = 0; c.ir = 1.f; c.absmax = 1.f; c.rs = 1.f; c.xrow = 0; c.dir_acc = 0.f; c.keep = 0; c.post = 1.f;
  if (!in_range) return c;
  c.dst = p.dst_row[i];
  if (c.dst < 0 || c.dst >= p.dst_rows) {
    report(p.status, AMOE_ERR_INDEX_RANGE, 10, static_cast<int>(i), static_cast<int>(c.dst));
    c.valid = 0;
    return c;
  }
  if (p.ir) c.ir = p.ir[i];
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

// Four consecutive columns n0..n0+3 (n0 % 4 == 0) of the row; v = raw accumulators.
__device__ __forceinline__ void epi_quad(const EpiParams& p, RowCtx& c, int n0, float v[4]) {
  if (!c.valid || n0 >= p.n_out) return;
  float o[4];
  float code[4] = {0.f, 0.f, 0.f, 0.f};
  if (!p.is_dx) {
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.noise_std > 0.f) {
      float4 zz = philox_normal4(p.seed, p.offset, kStreamOutNoise, static_cast<uint32_t>(c.dst),
                                 static_cast<uint32_t>(n0 >> 2));
      z[0] = zz.x; z[1] = zz.y; z[2] = zz.z; z[3] = zz.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + j;
      if (n < p.n_out) {
        float acc = v[j] * p.acc_mul;
        float s = (p.col_scale != nullptr) ? p.col_scale[static_cast<int64_t>(c.e) * p.n_out + n] : 1.f;
        if (p.noise) acc += p.noise[c.dst * p.n_out + n];
        if (p.noise_std > 0.f) acc += (p.noise_std * s) * z[j];
        if (p.adc.on) acc = (s > 0.f) ? adc_apply(acc, s, p.adc, code[j]) : 0.f;
        if (p.a_absmax) acc *= c.absmax;
        if (p.ir) acc *= c.ir;
        o[j] = acc;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + j;
      if (n < p.n_out) {
        float g = v[j];
        float gs = g * c.rs;
        if (p.x_ref) {
          float xr = load_elem(p.x_ref, p.x_ref_dtype, c.xrow * p.x_ref_stride + n);
          bool up = xr >= c.ir, low = xr <= -c.ir, keep = fabsf(xr) < c.ir;
          if (up) c.dir_acc += fminf(gs, 0.f);
          if (low) c.dir_acc -= fmaxf(gs, 0.f);
          c.keep += keep ? 1u : 0u;
          gs = keep ? gs : 0.f;
        }
        o[j] = gs;
      }
    }
  }
  const int64_t base = c.dst * p.out_stride + n0;
  if (n0 + 3 < p.n_out && p.out_dtype == AMOE_F32 && ((base & 3) == 0)) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + base) = make_float4(o[0], o[1], o[2], o[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n0 + j < p.n_out) store_elem(p.out, p.out_dtype, base + j, o[j]);
  }
  if (p.out_codes) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n0 + j < p.n_out) p.out_codes[c.dst * p.n_out + n0 + j] = static_cast<int8_t>(code[j]);
  }
}

// After the last column: per-row results of the input-gradient epilogue.
__device__ __forceinline__ void epi_row_end(const EpiParams& p, RowCtx& c, int64_t i) {
  if (!p.is_dx || !c.valid) return;
  if (p.ir_grad) {
    float d = c.dir_acc;
    if (p.relative) d = (d * c.ir) * p.grad_scale;
    p.ir_grad[i] = d;
  }
}

}  // namespace amoe
