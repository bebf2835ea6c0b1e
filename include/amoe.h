/*
 * amoe.h - C ABI of the B200 analog-CVMM library (libamoe_b200.so).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, runs
 * asynchronously on that stream and returns an `amoe_status`.  Unless a function's
 * comment says otherwise the library allocates nothing: the caller owns inputs,
 * outputs and the workspaces whose sizes the `*_workspace_bytes` helpers report.
 * Index arrays are int32.  Matrices are row-major with the row stride given in
 * elements.  "Slot" = one routed (token, expert) pair; slots are numbered
 * token*k + j ("flat slot") and are processed in expert-sorted order ("sorted
 * position").  P = T*k slots, E experts.
 *
 * The functions replace the Triton kernels and their wrappers in the reference's
 * analog_moe/triton_src/cvmm.py; each comment cites the lines it replaces.
 */
#ifndef AMOE_H_
#define AMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* amoe_stream_t; /* a cudaStream_t */

typedef enum amoe_status {
  AMOE_OK = 0,
  AMOE_ERR_BAD_SHAPE = 1,     /* a size is non-positive or violates a documented limit */
  AMOE_ERR_BAD_DTYPE = 2,
  AMOE_ERR_NULL_POINTER = 3,  /* a required pointer is NULL */
  AMOE_ERR_WORKSPACE = 4,     /* workspace missing or too small */
  AMOE_ERR_CUDA = 5,          /* a CUDA runtime/driver call failed; see amoe_last_error_string */
  AMOE_ERR_UNSUPPORTED = 6,   /* combination of options not implemented */
  AMOE_ERR_DEVICE = 7,        /* the current device is not an sm_100 part */
  AMOE_ERR_INDEX_RANGE = 8,   /* device-side check saw an index out of range (amoe_read_device_status) */
  AMOE_ERR_WAIT_LIMIT = 9     /* a bounded device-side wait gave up (amoe_read_device_status) */
} amoe_status;

typedef enum amoe_dtype { AMOE_F32 = 0, AMOE_BF16 = 1,
                          AMOE_F16 = 2   /* IEEE half: only where a function says so (amoe_operand_tiles, gradient rows) */
} amoe_dtype;

/* How the contraction is carried out. */
typedef enum amoe_precision {
  AMOE_PREC_BF16X1 = 0, /* one tcgen05 bf16 pass; exact when both operands are bf16-representable */
  AMOE_PREC_SPLIT = 1,  /* fp32 operands split into bf16 hi+lo terms, 2-3 tcgen05 passes, fp32 accumulate */
  AMOE_PREC_FP32_SIMT = 2, /* CUDA-core fp32 FMA (the arithmetic the reference's fp32 kernel uses) */
  AMOE_PREC_F16X1 = 3   /* fp32 data as IEEE fp16 operands (11-bit significands: ~2e-4 of the result's scale), one
                           tcgen05 pass, fp32 accumulate.  Integer DAC codes are exact.  Gradient operands are scaled
                           by a power of two taken from the tensor's largest magnitude (amoe_tensor_absmax) so that
                           they sit in fp16's normal range whatever their size; conversions saturate at +-65504.
                           The prepared weight copies and operand caches hold fp16 instead of bf16. */
} amoe_precision;

int amoe_version(void);
const char* amoe_status_string(int status);
/* Text of the last CUDA error this thread's calls ran into ("" if none). */
const char* amoe_last_error_string(void);
/* Number of kernels the calling thread's calls into this library have launched so far (every kernel of the
 * library is counted where it is launched; memsets and copies are not kernels and are not counted). */
unsigned long long amoe_launch_count(void);
/* AMOE_OK if the current CUDA device can run the kernels (compute capability 10.x). */
int amoe_check_device(void);

/* ------------------------------------------------------------------------------------------
 * Device status word.  Kernels never trap: an index outside its range or a bounded wait that
 * ran out is recorded in a caller-provided int32[4] {code, detail0, detail1, detail2} (may be
 * NULL to disable) and the offending access is skipped.  amoe_read_device_status copies it to
 * the host (synchronising the stream) and returns the amoe_status it encodes.
 * ---------------------------------------------------------------------------------------- */
int amoe_read_device_status(const int32_t* dev_status, int32_t host_copy[4], amoe_stream_t stream);

/* Exercises the give-up path of the kernels' bounded waits without stalling anything: a one-block kernel waits on a
 * barrier nobody arrives at, with a limit of `limit_cycles` GPU clock cycles (<= 4e9; a few million is a millisecond or
 * two), records AMOE_ERR_WAIT_LIMIT {where = 99} in dev_status and returns normally.  (No counterpart in the reference.) */
int amoe_selftest_bounded_wait(int32_t* dev_status, long long limit_cycles, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Routing.  Replaces the sigmoid/top-k of the sigma-MoE base layer (restated in the reference at
 * tests/test_moe_layer_aihwkit.py:71-76) and cvmm_prepare_sel's flatten+sort (cvmm.py:31-34).
 *
 * logits [T,E] fp32 -> raw_sel [T,k] (expert ids by descending gate value, lower id first on
 * ties), gate [T,k] (sigmoid(logit) if apply_sigmoid else logit), and the stable expert-sorted
 * slot list: sel_sorted [P], token_index [P] (= flat slot / k), slot_index [P] (flat slot),
 * expert_offsets [E+1].  E <= 1024, k <= 32, k <= E.  Workspace: amoe_select_sort_workspace_bytes.
 * ---------------------------------------------------------------------------------------- */
size_t amoe_select_sort_workspace_bytes(int64_t T, int32_t E, int32_t k);
int amoe_select_sort(const float* logits, int64_t T, int32_t E, int32_t k, int32_t apply_sigmoid,
                     int32_t* raw_sel, float* gate, int32_t* sel_sorted, int32_t* token_index,
                     int32_t* slot_index, int32_t* expert_offsets, void* workspace, size_t workspace_bytes,
                     amoe_stream_t stream);

/* The sort half of amoe_select_sort for a raw_sel [T,k] that already exists (workspace as for amoe_select_sort). */
int amoe_sort_slots(const int32_t* raw_sel, int64_t T, int32_t E, int32_t k, int32_t* sel_sorted, int32_t* token_index,
                    int32_t* slot_index, int32_t* expert_offsets, void* workspace, size_t workspace_bytes,
                    amoe_stream_t stream);

/* Backward of the gate selection: dlogits [T,E] = 0 except dlogits[t, raw_sel[t,j]] = dgate[t,j]*(1-g)*g with
 * g = gate[t,j] (apply_sigmoid) or dgate[t,j].  Replaces autograd's gather/sigmoid backward of the base layer's
 * `sigmoid(logits).gather(raw_sel)`; every element of dlogits is written. */
int amoe_gate_backward(const float* dgate, const float* gate, const int32_t* raw_sel, int64_t T, int32_t E, int32_t k,
                       int32_t apply_sigmoid, float* dlogits, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * The router around the path (the base layer's `F.linear(input, expert_sel.weight)`, restated in the reference at
 * tests/test_moe_layer_aihwkit.py:71-76, and its autograd backward).
 * amoe_router_logits: logits[t,e] = sum_d x[t,d]*w[e,d] (+ bias[e]), fp32 accumulate; round_bf16 rounds the result
 *   (and the sum with the bias) to bf16 the way a bf16 linear layer would.  w is [E,D] contiguous.
 * amoe_router_backward_w: dw_sel[e,:] = sum over the slots i of expert e of c_i * x[token_index[i],:], with
 *   c = dgate*(1-g)*g (apply_sigmoid) or dgate, dgate/gate indexed by flat slot (slot_index[i]).  Fixed summation order.
 *   raw_sel [T,k] (optional) enables a token-major variant that reads x once when the [E,D] gradient fits in shared memory.
 * amoe_combine_router: y[t,:] = sum_j res[row(t*k+j),:] + sum_j c[t,j] * w_sel[raw_sel[t,j],:] (row() as in
 *   amoe_combine): the sum over k of the
 *   up-projection's input gradient (cvmm.py:890-891) and the router's own input gradient in one pass.
 * ---------------------------------------------------------------------------------------- */
int amoe_router_logits(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const void* w,
                       int32_t w_dtype, int32_t E, const float* bias, int32_t round_bf16, float* logits,
                       amoe_stream_t stream);
/* amoe_router_select: amoe_router_logits with the gate selection in the same kernel (E <= 64, 16-byte aligned rows):
 *   raw_sel [T,k] and gate [T,k] as amoe_select_sort writes them; logits [T,E] optional.  Follow with amoe_sort_slots. */
int amoe_router_select(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const void* w,
                       int32_t w_dtype, int32_t E, const float* bias, int32_t round_bf16, int32_t k, int32_t apply_sigmoid,
                       float* logits, int32_t* raw_sel, float* gate, amoe_stream_t stream);
size_t amoe_router_backward_w_workspace_bytes(int64_t P, int32_t E, int32_t D);
int amoe_router_backward_w(const void* x, int32_t x_dtype, int64_t x_stride, int64_t T, int32_t D, const float* dgate,
                           const float* gate, int32_t apply_sigmoid, const int32_t* token_index,
                           const int32_t* slot_index, const int32_t* expert_offsets, const int32_t* raw_sel, int64_t P,
                           int32_t E, float* dw_sel, void* workspace, size_t workspace_bytes, amoe_stream_t stream);
int amoe_combine_router(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, int64_t T,
                        int32_t k, int32_t N,
                        const float* dgate, const float* gate, int32_t apply_sigmoid, const int32_t* raw_sel,
                        const void* w_sel, int32_t w_dtype, int32_t E, void* y, int32_t y_dtype, int64_t y_stride,
                        amoe_stream_t stream);

/* expert_offsets [E+1] from an already sorted expert-id list (a CVMMSel.sel built elsewhere). */
int amoe_expert_offsets(const int32_t* sel_sorted, int64_t P, int32_t E, int32_t* expert_offsets,
                        int32_t* dev_status, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Weight pre-pass.  Replaces modify_weight (moe_layer_aihwkit_lightning.py:313-382,
 * moe_layer_aihwkit.py:144-196) and the |W| maxima the layers take for the output noise
 * (moe_layer_aihwkit_lightning.py:480-487), and lays the weights out for the tensor cores.
 *
 * W [E,K,N] (strides in elements, any layout) -> col_scale [E,N] fp32 = per-column max|W|
 * (per_channel_scale) or the per-expert max broadcast; W' = discretise(W) + std*scale*z with z
 * Philox normals (seed, offset; element (e,k,n) = row e*K+k, column n of the weight stream);
 * then, for the tcgen05 kernels, bf16 "hi" (and "lo" = bf16(W' - hi) when requested) copies in two
 * K-major layouts, zero padded: `fwd_*` [E, Npad, Kpad] for x@W and `bwd_*` [E, Kpad2, Npad2]
 * for g@W^T, where Npad = roundup(N,16), Kpad = roundup(K,64), Kpad2 = roundup(K,16),
 * Npad2 = roundup(N,64) (amoe_prepared_dims).  `w_out` (optional, [E,K,N] fp32 contiguous) receives W' itself.
 * Any of the output pointers may be NULL.
 * ---------------------------------------------------------------------------------------- */
typedef struct amoe_weight_prepass_args {
  const void* w; int32_t w_dtype; int32_t E, K, N;
  int64_t w_stride_e, w_stride_k, w_stride_n;
  int32_t per_channel_scale;      /* 1: col_scale per column, 0: per expert */
  float noise_std;                /* <=0: no additive noise */
  int32_t noise_per_channel;      /* scale of the noise: per column (1) or per expert (0) maximum */
  float discretize_res;           /* <=0: off; else n_states = max(res, 1/res) */
  uint64_t seed; uint32_t offset;
  const long long* step_dev;      /* optional device counter: the Philox offset used is offset + 8 * (*step_dev) */
  float* col_scale;               /* [E,N] */
  float* col_inv_scale;           /* [E,N] correctly rounded 1/col_scale (0 where col_scale is 0), or NULL */
  float* w_out;                   /* [E,K,N] fp32 or NULL */
  void* fwd_hi; void* fwd_lo;     /* bf16 [E,Npad,Kpad] or NULL */
  void* bwd_hi; void* bwd_lo;     /* bf16 [E,Kpad2,Npad2] or NULL */
  void* workspace; size_t workspace_bytes;  /* amoe_weight_prepass_workspace_bytes (_clip_ with clipping) */
  /* Weight clipping in the same pass (clip_weights of the layers, moe_layer_aihwkit_lightning.py:519-543,
   * moe_layer_aihwkit.py:314-340): W is first clamped to +-bound, bound = clip_sigma * std (unbiased; of each column
   * over K if clip_per_channel, else of the whole expert), capped by clip_fixed when that is positive; clip_sigma <= 0
   * with clip_fixed > 0 clamps to +-clip_fixed.  The clamped weights are written to w_clip_out (same type and strides
   * as w; pass w itself to clip in place) and everything else - maxima, modifier, prepared copies - is computed from
   * them.  Needs the larger workspace of amoe_weight_prepass_clip_workspace_bytes (8-byte aligned). */
  float clip_sigma; int32_t clip_per_channel; float clip_fixed; void* w_clip_out;
  /* Added to the expert index in the weight-noise counter (row (expert_base + e)*K + k): a rank that holds experts
   * [base, base + E) of a larger layer draws the noise the whole layer would draw for them. */
  int32_t expert_base;
  int32_t prepared_f16;  /* non-zero: fwd_hi / bwd_hi receive IEEE fp16 (for AMOE_PREC_F16X1; lo pointers must be NULL) */
} amoe_weight_prepass_args;
size_t amoe_weight_prepass_workspace_bytes(int32_t E, int32_t K, int32_t N);
size_t amoe_weight_prepass_clip_workspace_bytes(int32_t E, int32_t K, int32_t N);
/* Padded extents of the prepared copies: dims[0..1] = {Npad, Kpad} (fwd), dims[2..3] = {Kpad2, Npad2} (bwd). */
void amoe_prepared_dims(int32_t K, int32_t N, int32_t dims[4]);
int amoe_weight_prepass(const amoe_weight_prepass_args* args, amoe_stream_t stream);

/* max|x| over the first n_rows rows of x [rows,K] into one device float (n_rows_dev: optional device int32 that holds
 * the row count, capped at rows; NULL = all rows).  NaNs are ignored.  The scalar that scales fp16 gradient operands. */
int amoe_tensor_absmax(const void* x, int32_t dtype, int64_t rows, int32_t K, int64_t stride, const int32_t* n_rows_dev,
                       float* absmax, amoe_stream_t stream);

/* |x| maximum of every row, x [R,K] -> absmax [R].  Replaces x.abs().amax(-1) (cvmm.py:733,737). */
int amoe_row_absmax(const void* x, int32_t dtype, int64_t R, int32_t K, int64_t stride, float* absmax,
                    amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * The conditional vector-matrix multiply.
 *
 * amoe_cvmm_fwd replaces cvmm_kernel + cvmm_triton_quantized (cvmm.py:37-231, 529-631) including
 * the noise the layers materialise (moe_layer_aihwkit_lightning.py:471-492), and adds the ADC:
 *   for sorted position i (expert e, source row r=a_row[i], destination row c=dst_row[i]):
 *     a   = A[r,:]; clamp to +-ir[i]; /ir[i]; /a_absmax[r]; round(a/inp_res)  (integer DAC code)
 *     acc = inp_res * sum_k code_k W'[e,k,:]             (fp32 accumulate)
 *     acc += noise[c,:]  |  noise_std*col_scale[e,:]*z(c,:)            (Philox, seed/offset; z(c,n): Philox4x32-10 with
 *            counter (c, n/8, 0x0A0E, offset) and key (seed lo, seed hi); output word j gives columns 8*(n/8)+2j, +2j+1 as
 *            r*cos(t), r*sin(t) with r = sqrt(-2 ln((lo16+0.5)/2^16)), t = 2 pi (hi16+0.5)/2^16 of the word's halves)
 *     ADC: q = rint(clamp(acc*(1/col_scale[e,:]), +-out_bound) * (1/step)), acc = q*step*col_scale[e,:]
 *     out[c,:] = acc * a_absmax[r] * ir[i];  out_codes[c,:] = q
 *
 * amoe_cvmm_dx replaces the second cvmm_triton_quantized call of CVMM.backward and the torch code
 * after it (cvmm.py:828-881): acc = G[r,:] @ W[e]^T (no DAC), then with x_ref/ir given
 *     up   = x_ref[xr,:] >= ir[i], low = x_ref[xr,:] <= -ir[i], keep = |x_ref[xr,:]| < ir[i]
 *     ir_grad[i] = (sum_n min(up*acc*rs,0) - sum_n max(low*acc*rs,0)) * (relative ? ir[i]*grad_scale : 1)
 *     out[c,:]   = keep * acc * rs        rs = row_scale[c] (the gate, down-projection) or 1
 *     keep_count += number of kept elements (for the decay term)
 *
 * Weights: `w` [E,K,N] fp32/bf16 with strides for AMOE_PREC_FP32_SIMT; the prepared bf16 copies
 * (see amoe_weight_prepass; fwd_* for amoe_cvmm_fwd, bwd_* for amoe_cvmm_dx) otherwise.
 * For amoe_cvmm_dx, K and N below are those of the *forward* weight [E,K,N]: A has N columns and
 * the result has K columns.
 * ---------------------------------------------------------------------------------------- */
typedef struct amoe_cvmm_args {
  int64_t P;                      /* sorted positions */
  int32_t E, K, N;                /* weight [E,K,N] */
  int32_t precision;              /* amoe_precision */
  const int32_t* expert_offsets;  /* [E+1] */
  const void* a; int32_t a_dtype; int64_t a_stride; int64_t a_rows;   /* input rows */
  const int32_t* a_row;           /* [P] source row of sorted position i ... */
  int32_t a_row_div;              /* ... divided by this (>=1; k folds the repeat of a token's row over its slots) */
  const int32_t* dst_row;         /* [P] destination row of sorted position i */
  int64_t dst_rows;               /* rows of out */
  /* weights */
  const void* w; int32_t w_dtype; int64_t w_stride_e, w_stride_k, w_stride_n;
  const void* w_hi; const void* w_lo;  /* prepared bf16 copies (lo may be NULL) */
  /* DAC */
  const float* ir;                /* [P] by sorted position, or NULL */
  int32_t ir_by_expert;           /* non-zero: ir holds E values, one per expert (no per-slot broadcast needed) */
  const float* a_absmax;          /* [a_rows] by source row, or NULL */
  float inp_res;                  /* <=0: no quantisation */
  /* output noise */
  const float* noise;             /* [dst_rows,N] fp32 by destination row, or NULL */
  float noise_std;                /* >0: Philox noise noise_std*col_scale[e,n]*z */
  uint64_t seed; uint32_t offset;
  const long long* step_dev;      /* optional device counter: the Philox offset used is offset + 8 * (*step_dev),
                                     so a captured CUDA graph draws fresh noise on every replay */
  const float* col_scale;         /* [E,N] (needed for Philox noise and ADC) */
  const float* col_inv_scale;     /* [E,N] from the weight pre-pass (needed for the ADC) */
  /* ADC */
  float out_res, out_bound;       /* out_res<=0: off */
  /* outputs */
  void* out; int32_t out_dtype; int64_t out_stride;   /* may be NULL when out_codes is given */
  int8_t* out_codes;              /* [dst_rows,N] or NULL */
  float* out_row_scale;           /* [dst_rows] or NULL: absmax*ir of the row, so that
                                     out[c,n] = ((code*step)*col_scale[e,n])*out_row_scale[c] */
  int32_t* out_row_expert;        /* [dst_rows] or NULL: expert of the row */
  int32_t out_relu;               /* amoe_cvmm_fwd: out = max(out, 0) (the activation between the projections) */
  /* backward-only (amoe_cvmm_dx) */
  const void* x_ref; int32_t x_ref_dtype; int64_t x_ref_stride; int64_t x_ref_rows;
  const int32_t* x_ref_row;       /* [P] row of x_ref for sorted position i */
  int32_t x_ref_relu;             /* amoe_cvmm_dx: additionally zero out[c,n] where x_ref <= 0 (backward of a ReLU
                                     that produced x_ref; applied after the input-range gradient is taken) */
  const float* row_scale;         /* [dst_rows] by destination row, or NULL */
  float* ir_grad;                 /* [P] by sorted position, or NULL */
  int32_t ir_grad_relative; float ir_grad_scale;
  unsigned long long* keep_count; /* one counter, incremented; or NULL */
  /* Operand caches for amoe_cvmm_dw (tensor-core precisions only; optional).  Rows are indexed by padded tile row:
   * the 128-row tiles of the expert-sorted slot list are numbered through all experts, tile t owns rows
   * [128t, 128t+128), rows past an expert's last slot are written as zeros.  Arrays are bf16, laid out as
   * [ceil(cols/64)][cache_rows][64] (64-column blocks, so that a 64 x 64 tile is one contiguous 8 KiB piece), with
   * cache_rows >= amoe_padded_rows(P,E); `lo` arrays hold the rounding residual of `hi` and may be NULL.
   *   a_cache_*  [rows, cols of A]: clamp(A[r,:], +-ir) * a_cache_scale[a_row[i]]   (needs cols % 8 == 0)
   *   out_cache_* (amoe_cvmm_dx) [rows, cols of out]: the result row                 (needs cols % 16 == 0)
   * No counterpart in the reference: its dW kernel re-reads and re-converts fp32 rows. */
  void* a_cache_hi; void* a_cache_lo; const float* a_cache_scale;
  void* out_cache_hi; void* out_cache_lo;
  int64_t cache_rows;
  /* The A operand itself as such a cache (bf16 hi, optional lo; cols % 64 == 0): when a_tile_hi is given the kernel
   * loads A through TMA, `a`/`a_row`/ir/a_absmax/inp_res are not used (whatever DAC the values need is already in
   * them) and no a_cache_* can be written.  amoe_cvmm_dx of an up-projection takes the out_cache of the
   * down-projection's amoe_cvmm_dx this way. */
  const void* a_tile_hi; const void* a_tile_lo;
  /* amoe_cvmm_fwd only: the result rows prepared as the NEXT projection's operands (same expert, e.g. the hidden
   * activation between up- and down-projection), by padded tile row, cols % 64 == 0:
   *   next_codes  bf16 DAC codes rint((clamp(out, +-next_ir[e]) / next_ir[e]) / next_inp_res): the next forward's a_tile_hi
   *   out_cache_* split(clamp(out, +-next_ir[e]) * out_cache_scale[dst row]): the next weight gradient's x operand
   * next_ir [E] per expert (required for next_codes; NULL = no clamp for out_cache_*). */
  const float* next_ir; float next_inp_res; void* next_codes; const float* out_cache_scale;
  /* plumbing */
  void* workspace; size_t workspace_bytes;  /* amoe_cvmm_workspace_bytes */
  int32_t* dev_status;            /* int32[4] or NULL */
  /* AMOE_PREC_F16X1, amoe_cvmm_dx: device scalar max|A| (amoe_tensor_absmax of the upstream gradient, or of the tensor
   * the A tiles were derived from).  With s = 2^k chosen so that max|A|*s lies in [2^7, 2^8): rows gathered from `a`
   * are multiplied by s before the conversion, A tiles (a_tile_hi) are taken to carry the factor s already, the
   * result is multiplied by 1/s, and out_cache_* keeps the result times s (so that it can serve as the next call's
   * A tiles and as a weight-gradient operand with the same scalar).  NULL: no scaling.
   * amoe_cvmm_dx accepts out == NULL when out_cache_hi is given (only the operand cache is wanted). */
  const float* a_absmax_dev;
} amoe_cvmm_args;
size_t amoe_cvmm_workspace_bytes(int64_t P, int32_t E);
/* Rows to allocate for an operand cache: (P/128 + E) * 128, an upper bound on the padded tile rows. */
int64_t amoe_padded_rows(int64_t P, int32_t E);
int amoe_cvmm_fwd(const amoe_cvmm_args* args, amoe_stream_t stream);
int amoe_cvmm_dx(const amoe_cvmm_args* args, amoe_stream_t stream);

/* Operand pre-pass: the A operand of amoe_cvmm_fwd / amoe_cvmm_dx as the tiles those calls take through a_tile_hi /
 * a_tile_lo, written by a streaming kernel of its own.  It is the top of the reference's matmul loop - load the
 * gathered row, clamp to +-ir, divide by ir and the abs-max, divide by the resolution, round (cvmm.py:139-172) - taken
 * out of the tensor-core kernel, where it runs on few threads and is latency-bound, into a pass that is HBM-bound.
 * Same arithmetic, same IEEE-exact quotients, same integer codes as the in-kernel path.
 *   dac != 0 (forward operand): tile = DAC codes (inp_res > 0) or the normalised rows, `cache` (optional) =
 *     clamp(A[r,:], +-ir) * cache_scale[a_row[i]]: the x operand of amoe_cvmm_dw from caches;
 *   dac == 0 (gradient operand): tile = the gathered rows converted (AMOE_PREC_F16X1: times the power of two derived
 *     from *g_absmax_dev, see amoe_cvmm_args.a_absmax_dev); the same array serves amoe_cvmm_dx as a_tile_hi and
 *     amoe_cvmm_dw as its g operand.  cache_hi must be NULL.
 * Element type of the arrays: IEEE fp16 for AMOE_PREC_F16X1, bf16 otherwise (`lo` arrays: bf16 rounding residuals,
 * AMOE_PREC_SPLIT only, may be NULL).  Layout [K/64][cache_rows][64] by padded tile row, rows past an expert's last
 * slot written as zeros; needs K % 64 == 0, 16-byte aligned rows, cache_rows >= amoe_padded_rows(P, E).
 * Source rows out of range are reported in dev_status (AMOE_ERR_INDEX_RANGE) and written as zeros. */
typedef struct amoe_operand_tiles_args {
  int64_t P; int32_t E; int32_t K;
  int32_t precision;              /* amoe_precision (not AMOE_PREC_FP32_SIMT) */
  const int32_t* expert_offsets;  /* [E+1] */
  const void* a; int32_t a_dtype; int64_t a_stride; int64_t a_rows;
  const int32_t* a_row; int32_t a_row_div;
  int32_t dac;
  const float* ir; int32_t ir_by_expert; const float* a_absmax; float inp_res;   /* as in amoe_cvmm_args */
  void* tile_hi; void* tile_lo;
  void* cache_hi; void* cache_lo; const float* cache_scale;
  int64_t cache_rows;
  const float* g_absmax_dev;
  int32_t* dev_status;
  /* dac == 0, AMOE_PREC_F16X1, a_dtype == AMOE_F16: the rows are fp16 already, row r scaled by the power of two that
   * amoe_cvmm_args.a_absmax_dev describes for a_row_absmax[r] (amoe_ep_put_f16 writes such rows).  Each row is rescaled
   * to the power of two of *g_absmax_dev (>= every a_row_absmax), which is exact: the tiles equal those made from the
   * fp32 rows.  [a_rows] by source row; NULL otherwise. */
  const float* a_row_absmax;
} amoe_operand_tiles_args;
int amoe_operand_tiles(const amoe_operand_tiles_args* args, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * dW.  Replaces cvmm_backward_kernel3 + cvmm_triton_backward (cvmm.py:234-397, 645-696) and the
 * outer product that feeds it in the down-projection (cvmm.py:789):
 *   dW[e] = sum_{i in e} clamp(X[x_row[i],:], +-ir[i])^T (x) (g_scale[g_row[i]] * G[g_src_row(i),:])
 * where g_src_row(i) = g_row[i] / g_div (g_div = k folds the repeat over the k slots of a token;
 * 1 otherwise).  One owner per output tile, no atomics: results do not depend on scheduling.
 * dW is fp32 [E,K,N] contiguous and is fully written (zeros for experts without slots).
 * With a workspace of amoe_cvmm_dw_workspace_bytes (optional; 0 bytes for small problems) the tensor-core
 * kernel cuts each expert's slots into segments, one work item per segment and tile, and sums the
 * partial tiles in segment order afterwards: same determinism, balanced under skewed routing.
 * ---------------------------------------------------------------------------------------- */
typedef struct amoe_dw_args {
  int64_t P; int32_t E, K, N; int32_t precision;
  const int32_t* expert_offsets;
  const void* x; int32_t x_dtype; int64_t x_stride; int64_t x_rows;
  const int32_t* x_row;           /* [P] */
  const float* ir;                /* [P] or NULL */
  int32_t ir_by_expert;           /* non-zero: ir holds E values, one per expert */
  const void* g; int32_t g_dtype; int64_t g_stride; int64_t g_rows;
  const int32_t* g_row;           /* [P] */
  int32_t g_div;                  /* >=1 */
  const float* g_scale;           /* indexed by g_row[i], or NULL */
  float* dw;                      /* [E,K,N] */
  /* Alternative inputs (tensor-core precisions): both operands as cached bf16 hi (+ lo) terms in padded tile-row
   * order (see amoe_cvmm_args).  With x_hi and g_hi given, x/g/x_row/g_row/ir/g_scale are not read: clamp and
   * scale are already in the caches.  Layout [ceil(cols/64)][cache_rows][64]; cache_rows >= amoe_padded_rows. */
  const void* x_hi; const void* x_lo; const void* g_hi; const void* g_lo; int64_t cache_rows;
  int64_t expected_rows;          /* 0, or the slot count to tune the segment size for when P is only an upper bound
                                     (buffers of worst-case size); the workspace then comes from
                                     amoe_cvmm_dw_workspace_bytes_tuned with the same two values */
  void* workspace; size_t workspace_bytes;  /* amoe_cvmm_dw_workspace_bytes, or NULL */
  int32_t* dev_status;
  /* AMOE_PREC_F16X1: device scalar max|g| (see amoe_cvmm_args.a_absmax_dev).  Gathered g rows are multiplied by the
   * power of two s derived from it, a g cache is taken to carry s already, and dW is multiplied by 1/s. */
  const float* g_absmax_dev;
} amoe_dw_args;
size_t amoe_cvmm_dw_workspace_bytes(int64_t P, int32_t E, int32_t K, int32_t N, int32_t precision);
size_t amoe_cvmm_dw_workspace_bytes_tuned(int64_t P, int64_t expected_rows, int32_t E, int32_t K, int32_t N,
                                          int32_t precision);
int amoe_cvmm_dw(const amoe_dw_args* args, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Reductions around the CVMM.
 * amoe_combine: y[t,:] = sum_j w[t*k+j] * res[row(t*k+j),:] in slot order (w NULL = 1), where
 *   row(s) = row_index[s] if row_index is given (rows kept in another order, e.g. expert-sorted), else s.  Replaces the
 *   gate-weighted reduction (cvmm.py:757-759), its backward (cvmm.py:888) and the sum over k of
 *   the up-projection's input gradient (cvmm.py:890-891).  With `codes` given instead of `res`
 *   the rows are rebuilt from ADC codes: codes*step*col_scale[raw_sel[slot],:]*row_mult[row(slot)]; codes and
 *   row_mult are indexed by row(slot) (row_index, or the slot itself), raw_sel / row_expert by slot.
 * amoe_row_dot: d[s] = res[row(s),:] . g[s/k,:]  (gate gradient, cvmm.py:889).
 * amoe_ir_grad_reduce: per-expert sum of the per-slot input-range gradients plus the decay term
 *   decay*ir_e*count_e*[keep_count/total > min_percentage] (cvmm.py:872-878 followed by autograd's
 *   index-add of input_range[ir_idx][sel]).  ir_grad_slot [P] sorted; out [E].  total = total_rows_dev[0]*cols when
 *   the device counter is given (e.g. rows summed over the ranks of an expert-parallel group), else total_elements
 *   when positive, else expert_offsets[E]*cols.
 * ---------------------------------------------------------------------------------------- */
int amoe_combine(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, const float* w,
                 int64_t T, int32_t k, int32_t N, void* y, int32_t y_dtype, int64_t y_stride, amoe_stream_t stream);
int amoe_combine_codes(const int8_t* codes, const float* col_scale, const int32_t* raw_sel, const float* row_mult,
                       float step, const float* w, int64_t T, int32_t k, int32_t N, void* y, int32_t y_dtype,
                       int64_t y_stride, const int32_t* row_index, amoe_stream_t stream);
int amoe_row_dot(const void* res, int32_t res_dtype, int64_t res_stride, const int32_t* row_index, const void* g,
                 int32_t g_dtype, int64_t g_stride, int64_t P, int32_t k, int32_t N, float* d, amoe_stream_t stream);
/* amoe_row_dot_codes: the same gate gradient with the rows given as ADC codes:
 *   d[s] = sum_n ((codes[s,n]*step)*col_scale[row_expert[s],n])*row_scale[s] * g[s/k,n]. */
int amoe_row_dot_codes(const int8_t* codes, const float* col_scale, const int32_t* row_expert, const float* row_scale,
                       float step, const void* g, int32_t g_dtype, int64_t g_stride, int64_t P, int32_t k, int32_t N,
                       float* d, const int32_t* row_index, amoe_stream_t stream);
int amoe_ir_grad_reduce(const float* ir_grad_slot, const int32_t* expert_offsets, const float* input_range,
                        int32_t E, float decay, float min_percentage, const unsigned long long* keep_count,
                        double total_elements, const long long* total_rows_dev, int32_t cols, float* out,
                        amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Per-expert standard deviation of the routed rows.  Replaces cvmm_std and its two kernels
 * (cvmm.py:400-526).  x [x_rows,K], x_row [P] by sorted position -> std [E] (NaN for experts without
 * rows, as in the reference).  Workspace: amoe_expert_std_workspace_bytes(E) bytes, which the call
 * clears itself.  A row index outside [0, x_rows) is recorded in dev_status (may be NULL) and skipped.
 * ---------------------------------------------------------------------------------------- */
size_t amoe_expert_std_workspace_bytes(int32_t E);
int amoe_expert_std(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows, const int32_t* x_row,
                    const int32_t* expert_offsets, int64_t P, int32_t E, float* std_out, void* workspace,
                    size_t workspace_bytes, int32_t* dev_status, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * amoe_expert_std_static: the same statistic as amoe_expert_std for callers that must not
 * allocate device memory.  (No counterpart in the reference.)
 *
 * Who needs it: a host that gave all of the GPU's memory to its own arena at start-up, so that a
 * later cudaMalloc - its own or a framework allocator's - would fail or would have to take memory
 * back from a running model; and code on a latency-critical path, where an allocation's implicit
 * device synchronisation is not acceptable.  Such callers own x, the index arrays and std_out, but
 * have no spare buffer to lend as a workspace.
 *
 * The accumulators live in an array that is part of the library image: 3 * 4096 doubles (96 KiB)
 * held by every GPU context that loads the library, for as long as it is loaded.  Limits and
 * rules that follow from that:
 *   - E <= 4096; a larger E returns AMOE_ERR_BAD_SHAPE and amoe_last_error_string says why;
 *   - no cudaMalloc/cudaFree and no allocating library routine is called; the call only clears
 *     the accumulators (the array keeps the previous call's contents) and launches kernels;
 *   - all calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *     (different streams without an ordering between them, or different host threads) race and
 *     return garbage.  Calls on one stream are safe back to back;
 *   - the first call on each device looks the array's device address up (with that device
 *     current).  Make that first call outside any stream capture.
 * Arguments and result are those of amoe_expert_std without the workspace pair.
 * ---------------------------------------------------------------------------------------- */
int amoe_expert_std_static(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows,
                           const int32_t* x_row, const int32_t* expert_offsets, int64_t P, int32_t E, float* std_out,
                           int32_t* dev_status, amoe_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Expert-parallel exchange helpers (no counterpart in the reference, which is single-GPU).
 * amoe_ep_pack gathers rows x[src_row[i] / src_div] (optionally times row_scale[src_row[i]]) of the
 * sorted slot list into a contiguous send buffer in sorted
 * order (so that each destination rank's experts form one contiguous block) and can apply the DAC
 * on the way: int8 codes + one fp32 scale per row instead of the raw rows.
 * amoe_ep_unpack scatters received rows back to their flat-slot rows.
 * ---------------------------------------------------------------------------------------- */
int amoe_ep_pack(const void* x, int32_t dtype, int64_t stride, int32_t K, const int32_t* src_row, int32_t src_div,
                 const float* row_scale, int64_t P, const float* ir, float inp_res, void* send_rows,
                 int8_t* send_codes, float* send_scale, amoe_stream_t stream);
/* Regrouping of an expert-parallel receive buffer by local expert.  The buffer holds, for source rank g = 0..G-1, that
 * source's rows for local experts 0..El-1 in order (recv_counts [G,El], R rows in total).  local_order [R]: row of the
 * buffer for each expert-sorted position (for e, for g); local_offsets [El+1].  G*El <= 4096. */
int amoe_ep_local_plan(const int32_t* recv_counts, int32_t G, int32_t El, int64_t R, int32_t* local_order,
                       int32_t* local_offsets, amoe_stream_t stream);
/* Device-driven exchange (no value is needed on the host, so a whole step can be captured in a CUDA graph).
 * amoe_ep_plan: from the all-gathered count matrix gathered[source][destination][local expert] (int32, [G,G,El]) to this
 *   rank's plan, amoe_ep_plan_ints(G,El) int32 values: [0] rows received R, [1] rows sent, then arrays of G: send_off,
 *   off_in, recv_off, back_off (block starts in this rank's sorted list / the destination's receive buffer / this rank's
 *   receive buffer / the source's sorted list), then recv_counts [G,El].
 * amoe_ep_local_plan_dev: amoe_ep_local_plan with counts and R taken from the plan; arrays sized for cap_rows.
 * amoe_ep_put: row x[src_row[i]/src_div] (* row_scale[src_row[i]]) of sorted position i is stored at its place in the
 *   receive buffer of the rank owning expert sel_sorted[i] (= sel_sorted[i]/El); peer_ptrs: device array of G base
 *   pointers (buffers of peer_rows rows of K elements, this rank's own included).  Plain stores, no waiting.
 * amoe_ep_put_back: the first R rows of `rows` (receive order) go back to their place in the source rank's buffer.
 * A plan that reports more rows than a buffer holds, or a row whose destination lies outside the peer's buffer, is
 * recorded in dev_status (AMOE_ERR_INDEX_RANGE; may be NULL) and the row is dropped, never written out of bounds.
 * amoe_ep_share: a small all-gather and a barrier in one launch, over peer memory.  This rank's `nbytes` (a multiple of 4,
 *   may be 0: barrier only) are stored into every rank's slot buffer, flags are exchanged, and the G payloads are copied
 *   to `gathered` [G, nbytes] (may be NULL).  slot_ptrs / flag_ptrs: device arrays of G base addresses of the ranks'
 *   slot buffers (2 * G * slot_bytes bytes each) and flag arrays (G uint32 each, zero before the first call); `epoch`: a
 *   device counter of this rank (zero before the first call; advanced by the call, so the launch can be replayed from a
 *   CUDA graph).  Every rank must make the same sequence of calls on the same buffers.  The wait for the other ranks is
 *   bounded: after spin_limit polls AMOE_ERR_WAIT_LIMIT goes to dev_status and the kernel returns.  Peer stores issued by
 *   earlier kernels of the calling stream are visible to the other ranks' kernels launched after their call returns. */
int64_t amoe_ep_plan_ints(int32_t G, int32_t El);
int amoe_ep_plan(const int32_t* gathered, int32_t rank, int32_t G, int32_t El, int32_t* plan, amoe_stream_t stream);
int amoe_ep_local_plan_dev(const int32_t* plan, int32_t G, int32_t El, int64_t cap_rows, int32_t* local_order,
                           int32_t* local_offsets, int32_t* dev_status, amoe_stream_t stream);
int amoe_ep_share(const void* payload, int64_t nbytes, const uint64_t* slot_ptrs, int64_t slot_bytes,
                  const uint64_t* flag_ptrs, uint32_t* epoch, int32_t rank, int32_t G, void* gathered,
                  int64_t spin_limit, int32_t* dev_status, amoe_stream_t stream);
/* amoe_ep_put for fp32 gradient rows of the AMOE_PREC_F16X1 precision: half the bytes over NVLink.  The row
 * v = row_scale * x[src_row/src_div] is stored as fp16(v * s), s the power of two (amoe_cvmm_args.a_absmax_dev) of its
 * own max|v|, and that maximum goes to the same row of a second set of buffers (scale_ptrs: [peer_rows] floats per rank)
 * for amoe_operand_tiles (a_row_absmax).  K % 8 == 0, rows 16-byte aligned. */
int amoe_ep_put_f16(const float* x, int64_t stride, int32_t K, int64_t x_rows, const int32_t* src_row, int32_t src_div,
                    const float* row_scale, int64_t P, const int32_t* sel_sorted, int32_t El, const int32_t* plan,
                    const uint64_t* peer_ptrs, const uint64_t* scale_ptrs, int32_t G, int64_t peer_rows,
                    int32_t* dev_status, amoe_stream_t stream);
int amoe_ep_put(const void* x, int32_t dtype, int64_t stride, int32_t K, int64_t x_rows, const int32_t* src_row,
                int32_t src_div, const float* row_scale, int64_t P, const int32_t* sel_sorted, int32_t El,
                const int32_t* plan, const uint64_t* peer_ptrs, int32_t G, int64_t peer_rows, int32_t* dev_status,
                amoe_stream_t stream);
int amoe_ep_put_back(const void* rows, int32_t dtype, int64_t stride, int32_t K, const int32_t* plan,
                     const uint64_t* peer_ptrs, int32_t G, int64_t cap_rows, int64_t peer_rows, int32_t* dev_status,
                     amoe_stream_t stream);
/* inv[idx[i]] = i for a permutation idx of 0..P-1. */
int amoe_invert_index(const int32_t* idx, int64_t P, int32_t* inv, amoe_stream_t stream);
int amoe_ep_unpack(const void* recv_rows, int32_t dtype, int32_t N, const int32_t* dst_row, int64_t P,
                   void* out, int64_t out_stride, amoe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AMOE_H_ */
