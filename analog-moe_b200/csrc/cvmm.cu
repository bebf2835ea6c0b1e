// C-ABI entry points of the conditional vector-matrix multiply: argument checks and dispatch.
#include "gemm_common.cuh"

using namespace amoe;

namespace {

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(const amoe_cvmm_args* a) {
  AMOE_REQUIRE(a != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->P > 0 && a->E > 0 && a->K > 0 && a->N > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->P < (int64_t{1} << 31) && a->E <= 65535, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->expert_offsets && a->dst_row && (a->out || a->out_codes || a->out_cache_hi), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE((a->a && a->a_row) || (a->a_tile_hi && a->precision != AMOE_PREC_FP32_SIMT), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->a_dtype == AMOE_F32 || a->a_dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE(a->out_dtype == AMOE_F32 || a->out_dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE((a->a_rows > 0 || a->a_tile_hi) && a->dst_rows > 0, AMOE_ERR_BAD_SHAPE);
  if (a->precision == AMOE_PREC_FP32_SIMT) {
    AMOE_REQUIRE(a->w != nullptr, AMOE_ERR_NULL_POINTER);
    AMOE_REQUIRE(a->w_dtype == AMOE_F32 || a->w_dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  } else if (a->precision == AMOE_PREC_BF16X1 || a->precision == AMOE_PREC_SPLIT || a->precision == AMOE_PREC_F16X1) {
    AMOE_REQUIRE(a->w_hi != nullptr, AMOE_ERR_NULL_POINTER);
  } else {
    return AMOE_ERR_UNSUPPORTED;
  }
  return AMOE_OK;
}

}  // namespace

extern "C" {

size_t amoe_cvmm_workspace_bytes(int64_t P, int32_t E) {
  (void)P; (void)E;
  return 0;  // the kernels find their tiles from expert_offsets; nothing is staged in global memory
}

int64_t amoe_padded_rows(int64_t P, int32_t E) {
  if (P <= 0 || E <= 0) return 0;
  return (P / 128 + E) * 128;
}

size_t amoe_cvmm_dw_workspace_bytes(int64_t P, int32_t E, int32_t K, int32_t N, int32_t precision) {
  if (precision == AMOE_PREC_FP32_SIMT || P <= 0 || E <= 0 || K <= 0 || N <= 0) return 0;
  return dw_tc_workspace_bytes(P, 0, E, K, N);
}

size_t amoe_cvmm_dw_workspace_bytes_tuned(int64_t P, int64_t expected_rows, int32_t E, int32_t K, int32_t N,
                                          int32_t precision) {
  if (precision == AMOE_PREC_FP32_SIMT || P <= 0 || E <= 0 || K <= 0 || N <= 0) return 0;
  return dw_tc_workspace_bytes(P, expected_rows, E, K, N);
}

int amoe_cvmm_fwd(const amoe_cvmm_args* a, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int s = check_common(a);
  if (s != AMOE_OK) return s;
  EpiParams e{};
  e.is_dx = 0; e.n_out = a->N;
  e.noise = a->noise; e.noise_std = a->noise_std; e.seed = a->seed; e.offset = a->offset; e.step_dev = a->step_dev;
  philox_key_schedule(a->seed, e.pkeys);
  e.col_scale = a->col_scale;
  e.col_inv_scale = a->col_inv_scale;
  e.adc = make_adc(a->out_res, a->out_bound);
  AMOE_REQUIRE(!e.adc.on || a->col_inv_scale != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!(e.adc.on || a->noise_std > 0.f) || a->col_scale != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!a->out_codes || e.adc.on, AMOE_ERR_UNSUPPORTED);
  if (e.adc.on) {
    float res = a->out_res > 1.f ? 1.f / a->out_res : a->out_res;
    AMOE_REQUIRE(!a->out_codes || res >= 1.f / 254.5f, AMOE_ERR_UNSUPPORTED);  // codes must fit int8
  }
  e.a_absmax = a->a_absmax; e.ir = a->ir; e.ir_by_expert = a->ir_by_expert; e.a_row = a->a_row; e.dst_row = a->dst_row;
  e.out_relu = a->out_relu;
  e.a_div = a->a_row_div < 1 ? 1 : a->a_row_div;
  e.a_rows = a->a_rows; e.dst_rows = a->dst_rows;
  e.acc_mul = 1.f;
  e.out = a->out; e.out_dtype = a->out_dtype; e.out_stride = a->out_stride; e.out_codes = a->out_codes;
  e.out_row_scale = a->out_row_scale; e.out_row_expert = a->out_row_expert;
  e.status = a->dev_status;
  e.vec4 = (a->N % 4 == 0) && al16(a->col_scale) && al16(a->col_inv_scale) && al16(a->noise) && al16(a->out) &&
           (a->out_stride % 4 == 0) && al16(a->out_codes);
  AMOE_REQUIRE(!(a->a_cache_hi || a->out_cache_hi) || a->precision != AMOE_PREC_FP32_SIMT, AMOE_ERR_UNSUPPORTED);
  e.out_cache_hi = reinterpret_cast<__nv_bfloat16*>(a->out_cache_hi);
  e.out_cache_lo = reinterpret_cast<__nv_bfloat16*>(a->out_cache_lo);
  e.out_cache_stride = a->cache_rows;
  e.next_ir = a->next_ir; e.next_res = a->next_inp_res; e.next_codes = reinterpret_cast<__nv_bfloat16*>(a->next_codes);
  e.out_cache_scale = a->out_cache_scale;
  AMOE_REQUIRE(!(a->out_cache_hi || a->next_codes) || (a->N % 16 == 0 && al16(a->out_cache_hi) && al16(a->out_cache_lo) && al16(a->next_codes)),
               AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(!a->next_codes || (a->next_ir && a->next_inp_res > 0.f && a->precision != AMOE_PREC_FP32_SIMT && a->out), AMOE_ERR_UNSUPPORTED);
  AMOE_REQUIRE(!a->out_cache_hi || a->out, AMOE_ERR_UNSUPPORTED);
  if (a->precision == AMOE_PREC_FP32_SIMT) return launch_cvmm_simt(a, false, e, stream);
  return launch_cvmm_tc(a, false, e, stream);
}

int amoe_cvmm_dx(const amoe_cvmm_args* a, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int s = check_common(a);
  if (s != AMOE_OK) return s;
  EpiParams e{};
  e.is_dx = 1; e.n_out = a->K;
  e.adc.on = false;
  e.ir = a->ir; e.ir_by_expert = a->ir_by_expert; e.a_row = a->a_row; e.dst_row = a->dst_row; e.a_rows = a->a_rows; e.dst_rows = a->dst_rows;
  e.x_ref_relu = a->x_ref_relu;
  e.a_div = a->a_row_div < 1 ? 1 : a->a_row_div;
  e.acc_mul = 1.f;
  e.out = a->out; e.out_dtype = a->out_dtype; e.out_stride = a->out_stride; e.out_codes = nullptr;
  e.x_ref = a->x_ref; e.x_ref_dtype = a->x_ref_dtype; e.x_ref_stride = a->x_ref_stride; e.x_ref_row = a->x_ref_row;
  e.x_ref_rows = a->x_ref_rows;
  AMOE_REQUIRE(!a->x_ref || (a->x_ref_row && (a->ir || a->x_ref_relu)), AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!a->x_ref_relu || a->x_ref, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(!a->x_ref || a->x_ref_rows > 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(!a->x_ref || a->x_ref_dtype == AMOE_F32 || a->x_ref_dtype == AMOE_BF16, AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE(!a->ir_grad || (a->x_ref && a->ir), AMOE_ERR_NULL_POINTER);
  e.row_scale = a->row_scale; e.ir_grad = a->ir_grad; e.relative = a->ir_grad_relative;
  e.grad_scale = a->ir_grad_scale; e.keep_count = a->keep_count;
  AMOE_REQUIRE(a->out != nullptr || (a->out_cache_hi != nullptr && a->precision != AMOE_PREC_FP32_SIMT), AMOE_ERR_NULL_POINTER);
  e.status = a->dev_status;
  e.vec4 = (a->K % 4 == 0) && al16(a->out) && (a->out_stride % 4 == 0) &&
           (!a->x_ref || (al16(a->x_ref) && a->x_ref_stride % 4 == 0));
  AMOE_REQUIRE(!(a->a_cache_hi || a->out_cache_hi) || a->precision != AMOE_PREC_FP32_SIMT, AMOE_ERR_UNSUPPORTED);
  e.out_cache_hi = reinterpret_cast<__nv_bfloat16*>(a->out_cache_hi);
  e.out_cache_lo = reinterpret_cast<__nv_bfloat16*>(a->out_cache_lo);
  e.out_cache_stride = a->cache_rows;
  AMOE_REQUIRE(!a->out_cache_hi || (a->K % 16 == 0 && al16(a->out_cache_hi) && al16(a->out_cache_lo)), AMOE_ERR_BAD_SHAPE);
  if (a->precision == AMOE_PREC_FP32_SIMT) return launch_cvmm_simt(a, true, e, stream);
  return launch_cvmm_tc(a, true, e, stream);
}

int amoe_cvmm_dw(const amoe_dw_args* a, amoe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  AMOE_REQUIRE(a != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->P > 0 && a->E > 0 && a->K > 0 && a->N > 0 && a->E <= 65535, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->P < (int64_t{1} << 31), AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->expert_offsets && a->dw, AMOE_ERR_NULL_POINTER);
  if (a->x_hi || a->g_hi) {
    AMOE_REQUIRE(a->x_hi && a->g_hi, AMOE_ERR_NULL_POINTER);
    AMOE_REQUIRE(a->precision != AMOE_PREC_FP32_SIMT, AMOE_ERR_UNSUPPORTED);
    AMOE_REQUIRE(a->cache_rows >= amoe_padded_rows(a->P, a->E) && a->K % 8 == 0 && a->N % 8 == 0, AMOE_ERR_BAD_SHAPE);
    return launch_dw_tc(a, stream);
  }
  AMOE_REQUIRE(a->x && a->x_row && a->g && a->g_row, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE((a->x_dtype == AMOE_F32 || a->x_dtype == AMOE_BF16) && (a->g_dtype == AMOE_F32 || a->g_dtype == AMOE_BF16),
               AMOE_ERR_BAD_DTYPE);
  AMOE_REQUIRE(a->x_rows > 0 && a->g_rows > 0 && a->g_div >= 1, AMOE_ERR_BAD_SHAPE);
  if (a->precision == AMOE_PREC_FP32_SIMT) return launch_dw_simt(a, stream);
  if (a->precision == AMOE_PREC_BF16X1 || a->precision == AMOE_PREC_SPLIT || a->precision == AMOE_PREC_F16X1)
    return launch_dw_tc(a, stream);
  return AMOE_ERR_UNSUPPORTED;
}

}  // extern "C"
