// Operand pre-pass: the rows of a CVMM operand, gathered in expert-sorted order, clamped / normalised / quantised by
// the DAC and written as the 128-row x 64-column tiles the tensor-core kernels load by TMA - plus, optionally, the
// clamped unquantised rows as the weight gradient's operand.
//
// The reference does this work at the top of its matmul loop (cvmm.py:139-172: load, clamp, divide by the input range
// and the abs-max, divide by the resolution, round).  Inside a tensor-core kernel that arithmetic runs on a few
// hundred threads per SM and is bound by their latency; as a streaming pass of its own it runs at full occupancy and
// is bound by HBM (one read of every gathered row, one 2-byte write per element and array).
//
// Layout written: [64-column block][padded row][64] 16-bit elements, padded row = 128 * tile + row in tile, where the
// 128-row tiles of the sorted slot list are numbered through all experts (a tile never straddles two experts).
// Rows of a tile past its expert's last slot are written as zeros: the weight gradient contracts over them.
#include "gemm_common.cuh"
#include "tc_ptx.cuh"

namespace amoe {
namespace {

using namespace tc;

constexpr int kRows = 128;        // rows per tile
constexpr int kColsPerBlock = 256;  // columns a thread block covers: 32 lanes x 8 elements
constexpr int kThreads = 256;

enum { kDacNone = 0, kDacNorm = 1, kDacQuant = 2 };

struct OperandParams {
  int64_t P;
  int E, K;
  const int32_t* offsets;
  const void* a; int64_t a_stride; int64_t a_rows;
  const int32_t* a_row; int a_div;
  const float* ir; int ir_by_expert;
  const float* a_absmax;
  float inp_res;
  uint16_t* tile_hi; uint16_t* tile_lo;
  uint16_t* cache_hi; uint16_t* cache_lo; const float* cache_scale;
  int64_t cache_rows;
  const float* g_absmax;
  const float* a_row_absmax;   // fp16 input rows: the maximum each row was scaled for
  int32_t* status;
};

__device__ __forceinline__ uint32_t cvt_bf16x2_(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <bool F16>
__device__ __forceinline__ uint32_t cvt2(float lo, float hi) { return F16 ? cvt_f16x2(lo, hi) : cvt_bf16x2_(lo, hi); }

// Eight values as one 16-byte store of 16-bit terms, and (bf16 only, `lo` given) the rounding residuals as a second.
template <bool F16>
__device__ __forceinline__ void store8(uint16_t* hi, uint16_t* lo, int64_t off, const float v[8]) {
  uint32_t h[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) h[x] = cvt2<F16>(v[2 * x], v[2 * x + 1]);
  *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
  if (!F16 && lo != nullptr) {
    uint32_t l[4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
      l[x] = cvt_bf16x2_(v[2 * x] - __uint_as_float(h[x] << 16), v[2 * x + 1] - __uint_as_float(h[x] & 0xffff0000u));
    *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// DAC of eight clamped values as packed pairs: ((a/ir)/absmax)/res with IEEE-exact quotients, then the integer code by
// adding and subtracting 1.5 * 2^23 (round to nearest even, exact for |code| < 2^22).  The same arithmetic as
// dac_code_clamped, two elements per instruction.
__device__ __forceinline__ void dac8(float v[8], bool has_ir, float ir, float rcp_ir, bool has_am, float am, float rcp_am,
                                     bool quant, float res, float rcp_res) {
  const f32x2 nir = pack2(-ir, -ir), yir = pack2(rcp_ir, rcp_ir);
  const f32x2 nam = pack2(-am, -am), yam = pack2(rcp_am, rcp_am);
  const f32x2 nres = pack2(-res, -res), yres = pack2(rcp_res, rcp_res);
  const f32x2 magic = pack2(12582912.f, 12582912.f), nmagic = pack2(-12582912.f, -12582912.f);
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    f32x2 t = pack2(v[2 * x], v[2 * x + 1]);
    if (has_ir) t = div_by_rcp2(t, nir, yir);
    if (has_am) t = div_by_rcp2(t, nam, yam);
    if (quant) {
      t = div_by_rcp2(t, nres, yres);
      t = add2(add2(t, magic), nmagic);
    }
    unpack2(t, v[2 * x], v[2 * x + 1]);
  }
}

// A_T: element type of the input rows - 0 bf16, 1 fp32, 2 fp16
template <int A_T>
__device__ __forceinline__ void load8(const void* base, int64_t elem_off, float v[8]) {
  if (A_T == 2) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem_off));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[x]));
      v[2 * x] = f.x; v[2 * x + 1] = f.y;
    }
  } else if (A_T == 1) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem_off);
    const float4 x = __ldg(q), y = __ldg(q + 1);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
  } else {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      v[2 * x] = __uint_as_float(w[x] << 16);
      v[2 * x + 1] = __uint_as_float(w[x] & 0xffff0000u);
    }
  }
}

// The rows of one warp: rows w, w + 8, ... of the tile, four or eight at a time (eight or sixteen 16-byte loads in flight
// per lane); lane l holds columns 8l .. 8l+7 of the block's column group.  IR / AM / CSC are compile-time copies of "input ranges
// given", "abs-max given", "cache scale given" (kept as run-time flags they turn into selects inside the unrolled
// element loops).
template <int DAC, int A_T, bool F16, bool IR, bool AM, bool CSC>
__device__ __forceinline__ void tile_rows(const OperandParams& p, int e, int row0, int rows, int64_t t, int w, int lane) {
  const int k = blockIdx.y * kColsPerBlock + lane * 8;
  const bool k_in = k < p.K;          // (all lanes stay for the shuffles; K % 64 == 0, so whole groups of 8 lanes leave)
  const float rcp_res = quant_rcp(p.inp_res);
  float g_mul = 1.f;
  if (DAC == kDacNone && F16 && p.g_absmax != nullptr) { float inv; g_mul = grad_pow2_scale(__ldg(p.g_absmax), inv); }
  constexpr bool kRowMul = DAC == kDacNone && A_T == 2;   // fp16 rows, each with a power-of-two scale of its own
  float ir_e = 1.f;
  if (IR && p.ir_by_expert) ir_e = p.ir[e];
  const int64_t blk = static_cast<int64_t>(k >> 6) * p.cache_rows + t * kRows;    // + row, then * 64 + column in block
  const int kin = k & 63;

  // Row parameters once per row, not once per lane: lane l < 16 prepares row w + 8 l of this warp (source row - an
  // integer division -, input range, abs-max and their correctly rounded reciprocals), the row loop fetches them by
  // shuffle.
  int m_src = -1;
  float m_ir = ir_e, m_am = 1.f, m_csc = 1.f;
  if (lane < 16) {
    const int r = w + 8 * lane;
    if (r < rows) {
      const int64_t i = static_cast<int64_t>(row0) + r;
      const int raw = p.a_row[i];
      const int s = p.a_div == 1 ? raw : raw / p.a_div;
      if (s < 0 || s >= p.a_rows) {
        if (blockIdx.y == 0) report(p.status, AMOE_ERR_INDEX_RANGE, 30, static_cast<int>(i), s);
      } else {
        m_src = s;
        if (kRowMul && p.a_row_absmax != nullptr) {
          // from the row's own power of two to the tensor's: a power of two <= 1, the product is exact
          float inv;
          grad_pow2_scale(p.a_row_absmax[s], inv);
          m_csc = g_mul * inv;
        }
        if (IR && !p.ir_by_expert) m_ir = p.ir[i];
        if (AM) m_am = p.a_absmax[s];
        if (CSC) m_csc = p.cache_scale[raw];
      }
    }
  }
  const float m_rcp_ir = IR ? __frcp_rn(m_ir) : 1.f, m_rcp_am = AM ? __frcp_rn(m_am) : 1.f;

  // rows per round: eight for the plain conversion (sixteen 16-byte loads in flight per lane hide the latency of
  // the gather), four where the DAC arithmetic needs the registers
  constexpr int kRpi = DAC == kDacNone ? 8 : 4;
#pragma unroll 1
  for (int it = 0; it < 16 / kRpi; ++it) {
    const int rb = w + 8 * kRpi * it;
    float v[kRpi][8];
    int src[kRpi];
    float irv[kRpi], rirv[kRpi], amv[kRpi], ramv[kRpi], csc[kRpi];
#pragma unroll
    for (int j = 0; j < kRpi; ++j) {
      const int l = kRpi * it + j;
      src[j] = __shfl_sync(0xffffffffu, m_src, l);
      irv[j] = IR ? __shfl_sync(0xffffffffu, m_ir, l) : 1.f;
      rirv[j] = IR ? __shfl_sync(0xffffffffu, m_rcp_ir, l) : 1.f;
      amv[j] = AM ? __shfl_sync(0xffffffffu, m_am, l) : 1.f;
      ramv[j] = AM ? __shfl_sync(0xffffffffu, m_rcp_am, l) : 1.f;
      csc[j] = (CSC || kRowMul) ? __shfl_sync(0xffffffffu, m_csc, l) : 1.f;
    }
#pragma unroll
    for (int j = 0; j < kRpi; ++j) {
      if (src[j] >= 0 && k_in) {
        load8<A_T>(p.a, static_cast<int64_t>(src[j]) * p.a_stride + k, v[j]);
      } else {
#pragma unroll
        for (int x = 0; x < 8; ++x) v[j][x] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < kRpi; ++j) {
      const int r = rb + 8 * j;
      const int64_t off = ((blk + r) << 6) + kin;
      if (!k_in) continue;
      if (DAC == kDacNone) {
        if (F16) {
          const float mul = kRowMul ? csc[j] : g_mul;
#pragma unroll
          for (int x = 0; x < 8; ++x) v[j][x] *= mul;
        }
        store8<F16>(p.tile_hi, p.tile_lo, off, v[j]);
      } else {
        if (IR) {
#pragma unroll
          for (int x = 0; x < 8; ++x) v[j][x] = clamp_ir(v[j][x], irv[j]);
        }
        if (p.cache_hi != nullptr) {
          if (CSC) {
            float c8[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) c8[x] = v[j][x] * csc[j];
            store8<F16>(p.cache_hi, p.cache_lo, off, c8);
          } else {
            store8<F16>(p.cache_hi, p.cache_lo, off, v[j]);
          }
        }
        if (p.tile_hi != nullptr) {
          // (a row that is not read holds zeros, whose code is zero)
          dac8(v[j], IR, irv[j], rirv[j], AM, amv[j], ramv[j], DAC == kDacQuant, p.inp_res, rcp_res);
          store8<F16>(p.tile_hi, p.tile_lo, off, v[j]);
        }
      }
    }
  }
}

// grid.x = row tile (an upper bound: blocks past the last tile return), grid.y = group of 256 columns.
template <int DAC, int A_T, bool F16>
__global__ void __launch_bounds__(kThreads, 3) operand_tiles_kernel(const OperandParams p) {
  __shared__ int s_tile[3];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t t = blockIdx.x;
  if (w == 0) {
    // tile t -> (expert, first sorted position, rows): prefix sum of the experts' tile counts, 32 experts per round
    int64_t base = 0;
    int fe = -1, row0 = 0, rows = 0;
    for (int e0 = 0; e0 < p.E && fe < 0; e0 += 32) {
      const int e = e0 + lane;
      int o0 = 0, o1 = 0;
      if (e < p.E) { o0 = p.offsets[e]; o1 = p.offsets[e + 1]; }
      const int nt = (o1 - o0 + kRows - 1) / kRows;
      int incl = nt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      const int64_t lo = base + incl - nt, hi = base + incl;
      const unsigned m = __ballot_sync(0xffffffffu, nt > 0 && t >= lo && t < hi);
      if (m) {
        const int src = __ffs(m) - 1;
        const int64_t lo_s = __shfl_sync(0xffffffffu, lo, src);
        const int o0_s = __shfl_sync(0xffffffffu, o0, src), o1_s = __shfl_sync(0xffffffffu, o1, src);
        fe = e0 + src;
        row0 = o0_s + static_cast<int>(t - lo_s) * kRows;
        rows = min(kRows, o1_s - row0);
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) { s_tile[0] = fe; s_tile[1] = row0; s_tile[2] = rows; }
  }
  __syncthreads();
  const int e = s_tile[0], row0 = s_tile[1], rows = s_tile[2];
  if (e < 0) return;
  if (DAC == kDacNone) {
    tile_rows<DAC, A_T, F16, false, false, false>(p, e, row0, rows, t, w, lane);
  } else {
    const bool ir = p.ir != nullptr, am = p.a_absmax != nullptr, csc = p.cache_scale != nullptr && p.cache_hi != nullptr;
#define AMOE_ROWS(IR, AM, CSC) tile_rows<DAC, A_T, F16, IR, AM, CSC>(p, e, row0, rows, t, w, lane)
    if (ir) {
      if (am) { if (csc) AMOE_ROWS(true, true, true); else AMOE_ROWS(true, true, false); }
      else { if (csc) AMOE_ROWS(true, false, true); else AMOE_ROWS(true, false, false); }
    } else {
      if (am) { if (csc) AMOE_ROWS(false, true, true); else AMOE_ROWS(false, true, false); }
      else { if (csc) AMOE_ROWS(false, false, true); else AMOE_ROWS(false, false, false); }
    }
#undef AMOE_ROWS
  }
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace
}  // namespace amoe

using namespace amoe;

extern "C" int amoe_operand_tiles(const amoe_operand_tiles_args* a, cudaStream_t stream) {
  AMOE_REQUIRE(a != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->P >= 0 && a->E >= 1 && a->K >= 64 && a->K % 64 == 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->precision == AMOE_PREC_BF16X1 || a->precision == AMOE_PREC_SPLIT || a->precision == AMOE_PREC_F16X1,
               AMOE_ERR_UNSUPPORTED);
  AMOE_REQUIRE(a->a != nullptr && a->a_row != nullptr && a->expert_offsets != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->a_dtype == AMOE_F32 || a->a_dtype == AMOE_BF16 || a->a_dtype == AMOE_F16, AMOE_ERR_BAD_DTYPE);
  // fp16 rows: pre-scaled gradient rows of the fp16 precision only
  AMOE_REQUIRE(a->a_dtype != AMOE_F16 || (a->dac == 0 && a->precision == AMOE_PREC_F16X1 && a->a_row_absmax && a->g_absmax_dev),
               AMOE_ERR_UNSUPPORTED);
  AMOE_REQUIRE(a->tile_hi != nullptr || a->cache_hi != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_REQUIRE(a->dac != 0 || (a->cache_hi == nullptr && a->tile_hi != nullptr), AMOE_ERR_UNSUPPORTED);
  const int esz = a->a_dtype == AMOE_F32 ? 4 : 2;
  AMOE_REQUIRE(aligned16(a->a) && (a->a_stride * esz) % 16 == 0, AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(aligned16(a->tile_hi) && aligned16(a->tile_lo) && aligned16(a->cache_hi) && aligned16(a->cache_lo),
               AMOE_ERR_BAD_SHAPE);
  AMOE_REQUIRE(a->cache_rows >= amoe_padded_rows(a->P, a->E), AMOE_ERR_BAD_SHAPE);
  if (a->P == 0) return AMOE_OK;
  int s = amoe_check_device();
  if (s != AMOE_OK) return s;
  const bool f16 = a->precision == AMOE_PREC_F16X1;
  OperandParams p{};
  p.P = a->P; p.E = a->E; p.K = a->K;
  p.offsets = a->expert_offsets;
  p.a = a->a; p.a_stride = a->a_stride; p.a_rows = a->a_rows;
  p.a_row = a->a_row; p.a_div = a->a_row_div < 1 ? 1 : a->a_row_div;
  p.ir = a->dac ? a->ir : nullptr; p.ir_by_expert = a->ir_by_expert;
  p.a_absmax = a->dac ? a->a_absmax : nullptr;
  p.inp_res = a->dac ? a->inp_res : -1.f;
  p.tile_hi = reinterpret_cast<uint16_t*>(a->tile_hi);
  p.tile_lo = f16 ? nullptr : reinterpret_cast<uint16_t*>(a->tile_lo);
  p.cache_hi = reinterpret_cast<uint16_t*>(a->cache_hi);
  p.cache_lo = f16 ? nullptr : reinterpret_cast<uint16_t*>(a->cache_lo);
  p.cache_scale = a->cache_scale;
  p.cache_rows = a->cache_rows;
  p.g_absmax = a->g_absmax_dev;
  p.a_row_absmax = a->a_dtype == AMOE_F16 ? a->a_row_absmax : nullptr;
  p.status = a->dev_status;
  const int64_t max_tiles = a->P / kRows + a->E;
  AMOE_REQUIRE(max_tiles < (1ll << 31), AMOE_ERR_BAD_SHAPE);
  const dim3 grid(static_cast<unsigned>(max_tiles), static_cast<unsigned>((a->K + kColsPerBlock - 1) / kColsPerBlock));
  const int dac = !a->dac ? kDacNone : (a->inp_res > 0.f ? kDacQuant : kDacNorm);
  const bool f32 = a->a_dtype == AMOE_F32;
#define AMOE_OPERAND(DAC, F32, F16) operand_tiles_kernel<DAC, F32, F16><<<grid, kThreads, 0, stream>>>(p)
#define AMOE_OPERAND_DT(DAC)                                                   \
  do {                                                                         \
    if (f16) { if (f32) AMOE_OPERAND(DAC, true, true); else AMOE_OPERAND(DAC, false, true); }   \
    else { if (f32) AMOE_OPERAND(DAC, true, false); else AMOE_OPERAND(DAC, false, false); }     \
  } while (0)
  if (a->a_dtype == AMOE_F16) operand_tiles_kernel<kDacNone, 2, true><<<grid, kThreads, 0, stream>>>(p);
  else if (dac == kDacNone) AMOE_OPERAND_DT(kDacNone);
  else if (dac == kDacQuant) AMOE_OPERAND_DT(kDacQuant);
  else AMOE_OPERAND_DT(kDacNorm);
#undef AMOE_OPERAND_DT
#undef AMOE_OPERAND
  AMOE_LAUNCH_CHECK("operand_tiles");
  return AMOE_OK;
}
