// CUDA-core fp32 CVMM kernels (AMOE_PREC_FP32_SIMT): the arithmetic of the reference's fp32 path
// (individually rounded fp32 FMAs, cvmm.py:181 with allow_tf32=False), used as the exact mode and
// as the on-device cross-check of the tcgen05 kernels.
#include "epilogue.cuh"
#include "gemm_common.cuh"

namespace amoe {
namespace {

constexpr int kTM = 64, kTN = 64, kTKs = 16;

struct SimtParams {
  int64_t P; int E, Kc, Nout;          // contraction length, output columns
  const int32_t* offsets;
  const void* a; int a_dtype; int64_t a_stride; int64_t a_rows; const int32_t* a_row; int a_div;
  const void* w; int w_dtype; int64_t se, sk, sn;  // B[k][n] = w[e*se + k*sk + n*sn]
  const float* ir; const float* a_absmax; float inp_res; int dac;  // dac: apply clamp/scale(/quantise) to A
  EpiParams epi;
};

__global__ void __launch_bounds__(256) cvmm_simt_kernel(SimtParams p) {
  __shared__ float As[kTKs][kTM + 4];
  __shared__ float Bs[kTKs][kTN + 4];
  __shared__ float Cs[kTM][kTN + 1];
  __shared__ int s_tile[3];
  const int tid = threadIdx.x;
  if (tid == 0) {
    int e, row0, rows;
    find_tile(p.offsets, p.E, kTM, blockIdx.x, e, row0, rows);
    s_tile[0] = e; s_tile[1] = row0; s_tile[2] = rows;
  }
  __syncthreads();
  const int e = s_tile[0], row0 = s_tile[1], rows = s_tile[2];
  if (e < 0) return;

  // A-load role: row lr, 4 consecutive k
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int64_t li = static_cast<int64_t>(row0) + lr;
  bool l_ok = lr < rows;
  int64_t l_src = 0;
  float l_ir = 1.f, l_am = 1.f, l_rir = 1.f, l_ram = 1.f;
  const float rcp_res = quant_rcp(p.inp_res);
  const bool has_ir = p.dac && p.ir != nullptr, has_am = p.dac && p.a_absmax != nullptr;
  const bool quant = p.dac && p.inp_res > 0.f;
  if (l_ok) {
    l_src = p.a_row[li] / p.a_div;
    if (l_src < 0 || l_src >= p.a_rows) {
      report(p.epi.status, AMOE_ERR_INDEX_RANGE, 20, static_cast<int>(li), static_cast<int>(l_src));
      l_ok = false;
    } else {
      if (has_ir) { l_ir = p.ir[p.epi.ir_by_expert ? e : li]; l_rir = __frcp_rn(l_ir); }
      if (has_am) { l_am = p.a_absmax[l_src]; l_ram = __frcp_rn(l_am); }
    }
  }
  // B-load role
  const int bk = tid >> 4, bn = (tid & 15) * 4;
  // compute role
  const int ty = tid >> 4, tx = tid & 15;
  // row-owner role
  RowCtx ctx;
  if (tid < kTM) {
    ctx = epi_row_begin(p.epi, static_cast<int64_t>(row0) + tid, e, tid < rows);
    epi_row_side_outputs(p.epi, ctx);
  }

  for (int n0 = 0; n0 < p.Nout; n0 += kTN) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < p.Kc; k0 += kTKs) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = k0 + lk + j;
        float v = 0.f;
        if (l_ok && k < p.Kc) {
          v = load_elem(p.a, p.a_dtype, l_src * p.a_stride + k);
          if (p.dac) {
            if (quant)
              v = dac_code(v, has_ir, l_ir, l_rir, has_am, l_am, l_ram, p.inp_res, rcp_res) * p.inp_res;
            else
              v = dac_normalise(v, has_ir, l_ir, l_rir, has_am, l_am, l_ram);
          }
        }
        As[lk + j][lr] = v;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = k0 + bk, n = n0 + bn + j;
        float v = 0.f;
        if (k < p.Kc && n < p.Nout) v = load_elem(p.w, p.w_dtype, e * p.se + k * p.sk + n * p.sn);
        Bs[bk][bn + j] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kTKs; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) Cs[ty * 4 + i][tx * 4 + j] = acc[i][j];
    __syncthreads();
    if (tid < kTM) {
      for (int q = 0; q < kTN / 4; ++q) {
        float v[4] = {Cs[tid][q * 4], Cs[tid][q * 4 + 1], Cs[tid][q * 4 + 2], Cs[tid][q * 4 + 3]};
        epi_quad(p.epi, ctx, n0 + q * 4, v);
      }
    }
    __syncthreads();
  }
  if (tid < kTM) {
    epi_row_end(p.epi, ctx, static_cast<int64_t>(row0) + tid);
    if (p.epi.is_dx && p.epi.keep_count) {
      unsigned kc = ctx.valid ? ctx.keep : 0u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) kc += __shfl_xor_sync(0xffffffffu, kc, o);
      if ((tid & 31) == 0 && kc) atomicAdd(p.epi.keep_count, static_cast<unsigned long long>(kc));
    }
  }
}

struct SimtDwParams {
  int E, K, N;
  const int32_t* offsets;
  const void* x; int x_dtype; int64_t x_stride; int64_t x_rows; const int32_t* x_row; const float* ir; int ir_by_expert;
  const void* g; int g_dtype; int64_t g_stride; int64_t g_rows; const int32_t* g_row; int g_div;
  const float* g_scale;
  float* dw;
  int32_t* status;
};

__global__ void __launch_bounds__(256) dw_simt_kernel(SimtDwParams p) {
  __shared__ float As[kTKs][kTM + 4];
  __shared__ float Bs[kTKs][kTN + 4];
  const int tid = threadIdx.x;
  const int e = blockIdx.z, k0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int beg = p.offsets[e], end = p.offsets[e + 1];
  const int ty = tid >> 4, tx = tid & 15;
  // load roles: slot ls (0..15), 4 consecutive columns
  const int ls = tid >> 4, lc = (tid & 15) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int s0 = beg; s0 < end; s0 += kTKs) {
    const int i = s0 + ls;
    bool ok = i < end;
    int64_t xr = 0, gr = 0;
    float ir = 0.f, gs = 1.f;
    if (ok) {
      xr = p.x_row[i];
      gr = p.g_row[i];
      if (xr < 0 || xr >= p.x_rows || gr < 0 || gr / p.g_div >= p.g_rows) {
        report(p.status, AMOE_ERR_INDEX_RANGE, 30, i, static_cast<int>(xr));
        ok = false;
      } else {
        if (p.ir) ir = p.ir[p.ir_by_expert ? e : i];
        if (p.g_scale) gs = p.g_scale[gr];
        gr /= p.g_div;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = 0.f, b = 0.f;
      if (ok) {
        if (k0 + lc + j < p.K) {
          a = load_elem(p.x, p.x_dtype, xr * p.x_stride + k0 + lc + j);
          if (p.ir) a = clamp_ir(a, ir);
        }
        if (n0 + lc + j < p.N) b = gs * load_elem(p.g, p.g_dtype, gr * p.g_stride + n0 + lc + j);
      }
      As[ls][lc + j] = a;
      Bs[ls][lc + j] = b;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTKs; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i2 = 0; i2 < 4; ++i2) a[i2] = As[kk][ty * 4 + i2];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i2 = 0; i2 < 4; ++i2)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i2][j] = fmaf(a[i2], b[j], acc[i2][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (k < p.K && n < p.N) p.dw[(static_cast<int64_t>(e) * p.K + k) * p.N + n] = acc[i][j];
    }
}

}  // namespace

int launch_cvmm_simt(const amoe_cvmm_args* a, bool is_dx, const EpiParams& epi, cudaStream_t stream) {
  SimtParams p;
  p.P = a->P; p.E = a->E;
  p.offsets = a->expert_offsets;
  p.a = a->a; p.a_dtype = a->a_dtype; p.a_stride = a->a_stride; p.a_rows = a->a_rows; p.a_row = a->a_row;
  p.a_div = a->a_row_div < 1 ? 1 : a->a_row_div;
  p.w = a->w; p.w_dtype = a->w_dtype;
  p.se = a->w_stride_e;
  if (!is_dx) {
    p.Kc = a->K; p.Nout = a->N; p.sk = a->w_stride_k; p.sn = a->w_stride_n;
    p.ir = a->ir; p.a_absmax = a->a_absmax; p.inp_res = a->inp_res; p.dac = 1;
  } else {
    p.Kc = a->N; p.Nout = a->K; p.sk = a->w_stride_n; p.sn = a->w_stride_k;
    p.ir = nullptr; p.a_absmax = nullptr; p.inp_res = -1.f; p.dac = 0;
  }
  p.epi = epi;
  p.epi.acc_mul = 1.f;
  const int64_t tiles = (a->P + kTM - 1) / kTM + a->E;
  cvmm_simt_kernel<<<static_cast<unsigned>(tiles), 256, 0, stream>>>(p);
  AMOE_LAUNCH_CHECK("cvmm_simt");
  return AMOE_OK;
}

int launch_dw_simt(const amoe_dw_args* a, cudaStream_t stream) {
  SimtDwParams p;
  p.E = a->E; p.K = a->K; p.N = a->N; p.offsets = a->expert_offsets;
  p.x = a->x; p.x_dtype = a->x_dtype; p.x_stride = a->x_stride; p.x_rows = a->x_rows; p.x_row = a->x_row;
  p.ir = a->ir; p.ir_by_expert = a->ir_by_expert;
  p.g = a->g; p.g_dtype = a->g_dtype; p.g_stride = a->g_stride; p.g_rows = a->g_rows; p.g_row = a->g_row;
  p.g_div = a->g_div < 1 ? 1 : a->g_div; p.g_scale = a->g_scale;
  p.dw = a->dw; p.status = a->dev_status;
  dim3 grid((a->N + kTN - 1) / kTN, (a->K + kTM - 1) / kTM, a->E);
  dw_simt_kernel<<<grid, 256, 0, stream>>>(p);
  AMOE_LAUNCH_CHECK("dw_simt");
  return AMOE_OK;
}

}  // namespace amoe
