// Dense GEMM for sm_100a: TMA-fed tcgen05.mma with fp32 (or int32)
// accumulators in tensor memory.
//
//   C[b] = epilogue( alpha * op(A[b]) * op(B[b]) )        b = 0..batch-1
//
// op(A) is M x K, op(B) is K x N.  transA = 0: A stored row-major M x K
// (K-major operand); transA = 1: A stored K x M (MN-major operand).  transB = 1:
// B stored N x K (K-major, the "x @ W^T" form); transB = 0: B stored K x N
// (MN-major).  The four combinations cover forward, data-gradient and
// weight-gradient GEMMs without a transposed copy, like the trans flags of the
// reference's Gemm contract (backend/backend.go:61-78) that its MatMul backward
// relies on (tensor/ops_matmul.go:36-46).
//
// Two persistent kernels share one epilogue.
// One-CTA kernel (one CTA per SM, 320 threads, 128 x 256 or 128 x 128 tiles):
//   warp 0     TMA producer: one elected thread fills a ring of shared-memory stages
//   warp 1     MMA issuer: one elected thread runs the whole tcgen05.mma issue loop and
//              commits to mbarriers (an issue loop spread over a warp with `lane == 0`
//              branches left the tensor pipe idle a fifth of the time)
//   warps 2-9  epilogue: tcgen05.ld the accumulator, bias / activation / auxiliary tensor,
//              then a swizzled staging buffer per warp and TMA stores (direct 16-byte
//              stores remain for unaligned outputs and accumulation into C)
// Two-CTA kernel (a cluster of two CTAs per 256 x 256 tile, tcgen05 cta_group::2): each CTA
// stages its own rows of A and half of the columns of B; the leader issues the MMAs.
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the MMAs of tile
// i+1.  Split-K: K slices of a tile run as separate work units into fp32 partials that a
// finish kernel adds in slice order.
#include "common.cuh"

using namespace gb;

namespace {

constexpr int BM = 128;
constexpr int kSwizzleBytes = 128;  // one swizzle atom along the contiguous dim
constexpr int kMaxThreads = 64 + 32 * 8;

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_GELU_ERF = 3 };
enum AuxMode : int {
  AUX_NONE = 0,
  AUX_ADD = 1,          // out += aux (residual), after the activation
  AUX_STORE_PRE = 2,    // aux = pre-activation value (aux is an output)
  AUX_MUL_DGELU_TANH = 3,  // out *= gelu_tanh'(aux)
  AUX_MUL_DRELU = 4,       // out *= (aux > 0)
  AUX_MUL_DGELU_ERF = 5,   // out *= gelu_erf'(aux)
};
enum OutKind : int { OUT_BF16 = 0, OUT_F16 = 1, OUT_F32 = 2 };

struct GemmArgs {
  int M, N, K, batch;
  int num_m, num_n;
  void* C;
  const void* bias;  // fp32 or same 16-bit type as the inputs, length N
  void* aux;         // same 16-bit type as inputs, M x N
  long long ldc, ldaux, strideC, strideAux;
  int bias_f32;
  int act, aux_mode, out_kind, beta;
  float alpha;
  // int8 path: y = sx * sw[n] * (acc - zx * rowsum[n]) + bias[n]
  const float* q_sx;      // device scalar
  const int* q_zx;        // device scalar
  const float* q_sw;      // per-channel [N] or single value
  const int* q_rowsum;    // [N]
  int q_per_channel;
  int in_bf16;  // 1 = bf16 inputs, 0 = fp16 inputs (ignored for int8)
  int bcastA, bcastB;  // operand shared by every batch entry (batch stride 0)
  int group_m;         // row blocks per rasterisation group
  int tma_epi;         // 1: results leave through shared memory and TMA stores (16-bit outputs)
  int splits, kb_per;  // split-K: slice s of a tile covers k-blocks [s * kb_per, (s + 1) * kb_per)
  int* status;
};

template <int ESZ, int BN>
struct Cfg {
  static constexpr int BK = kSwizzleBytes / ESZ;  // elements per k-block
  static constexpr int UMMA_K = 32 / ESZ;
  static constexpr int A_BYTES = BM * kSwizzleBytes;
  static constexpr int B_BYTES = BN * kSwizzleBytes;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
};

// Dynamic shared memory of both kernels (the base must be 1024-byte aligned, which the
// kernels check):  [operand ring] [epilogue staging: 2 x 2 KB per epilogue warp, 16-bit
// path only] [512 B of barriers] [per-column epilogue constants, double buffered].
template <int ESZ, int RING, int EW>
struct SmemLayout {
  static constexpr int kStageBuf = 2048;  // 32 rows x 64 B, 64-byte swizzle
  static constexpr int OFF_STAGING = RING;
  static constexpr int STAGING = ESZ == 2 ? EW * 2 * kStageBuf : 0;
  static constexpr int OFF_BARS = OFF_STAGING + STAGING;
  static constexpr int OFF_COLS = OFF_BARS + 512;
  static constexpr int COL_BYTES = (ESZ == 1 ? 3 : 1) * 2 * 256 * 4;
  static constexpr int BYTES = OFF_COLS + COL_BYTES;
  static_assert(BYTES <= 232448, "shared memory layout exceeds 227 KB");
};

// Tile order: groups of `gm` row blocks are swept across all column blocks before the
// next group starts, so that the CTAs running at the same time share A and B tiles in L2.
__device__ __forceinline__ void tile_coords(int r, int num_m, int num_n, int gm, int& mb, int& nb) {
  const int per_group = gm * num_n;
  const int g = r / per_group;
  const int first = g * gm;
  const int rows = min(gm, num_m - first);
  const int in_g = r - g * per_group;
  mb = first + in_g % rows;
  nb = in_g / rows;
}

// Work unit t of a launch -> K slice, batch entry and tile coordinates.  Slices are the
// slowest index, so the CTAs first sweep slice 0 of every tile, then slice 1, ...
struct Unit {
  int s, b, mb, nb;
};
__device__ __forceinline__ Unit decode_unit(int t, const GemmArgs& args) {
  const int tiles_per_batch = args.num_m * args.num_n;
  const int per_slice = tiles_per_batch * args.batch;
  Unit u;
  u.s = t / per_slice;
  const int t2 = t - u.s * per_slice;
  u.b = t2 / tiles_per_batch;
  tile_coords(t2 - u.b * tiles_per_batch, args.num_m, args.num_n, args.group_m, u.mb, u.nb);
  return u;
}

template <typename T>
__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
    case ACT_RELU: return v > 0.f ? v : 0.f;
    case ACT_GELU_TANH: return gelu_tanh_f(v);
    case ACT_GELU_ERF: return gelu_erf_f(v);
    default: return v;
  }
}

__device__ __forceinline__ float2 unpack16(uint32_t u, int in_bf16) {
  return in_bf16 ? unpack_bf16(u) : unpack_f16(u);
}
__device__ __forceinline__ uint32_t pack16x(float a, float b, int bf) {
  return bf ? pack_bf16(a, b) : pack_f16(a, b);
}

// Per-warp constants of the epilogue.
struct EpiCtx {
  int q, half, et, lane;
  bool vec_ok, aux_vec_ok, aux_in, has_cols;
  float q_sx;
  int q_zx;
  float* s_bias;
  float* s_qsw;
  int* s_qrs;
};

template <int ESZ>
__device__ __forceinline__ EpiCtx make_epi_ctx(const GemmArgs& args, int warp, int lane, int et, float* s_bias,
                                               float* s_qsw, int* s_qrs) {
  EpiCtx c;
  c.q = warp & 3;
  c.half = (warp - 2) >> 2;
  c.et = et;
  c.lane = lane;
  c.vec_ok = ((args.ldc & 7) == 0) && ((args.strideC & 7) == 0) && (((uintptr_t)args.C & 15) == 0);
  c.aux_vec_ok = args.aux_mode == AUX_NONE || (((args.ldaux & 7) == 0) && ((args.strideAux & 7) == 0) &&
                                               (((uintptr_t)args.aux & 15) == 0));
  c.aux_in = args.aux_mode != AUX_NONE && args.aux_mode != AUX_STORE_PRE;
  c.has_cols = args.bias != nullptr || ESZ == 1;
  c.q_sx = 1.f;
  c.q_zx = 0;
  if (ESZ == 1) {
    c.q_sx = *args.q_sx;
    c.q_zx = args.q_zx ? *args.q_zx : 0;
  }
  c.s_bias = s_bias; c.s_qsw = s_qsw; c.s_qrs = s_qrs;
  return c;
}

// Epilogue of one 128-row x BN-column accumulator held in this CTA's TMEM at column
// `tmem_acc`: everything that does not depend on the accumulator (bias, residual / saved
// pre-activation) is fetched BEFORE waiting for the MMAs, so those latencies overlap the
// main loop of the tile.  Returns false when the wait ran out of budget.
template <int ESZ, int BN, int EW>
__device__ __forceinline__ bool epilogue_tile(const GemmArgs& args, const EpiCtx& cx, int buf, int b, int m0,
                                              int n0, uint32_t tmem_acc, uint64_t* tfull, uint32_t tfull_phase,
                                              volatile int* abort_flag) {
  constexpr int COLS = BN / (EW / 4);  // columns per thread per tile
  constexpr int NCH = COLS / 32;
  const int q = cx.q, half = cx.half, et = cx.et, lane = cx.lane;
  const bool vec_ok = cx.vec_ok, aux_vec_ok = cx.aux_vec_ok, aux_in = cx.aux_in, has_cols = cx.has_cols;
  const float q_sx = cx.q_sx;
  const int q_zx = cx.q_zx;
  float* s_bias = cx.s_bias;
  float* s_qsw = cx.s_qsw;
  int* s_qrs = cx.s_qrs;
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < args.M;
    const int cbase = n0 + half * COLS;  // first column of this thread
    // ---- per-column constants into shared memory (double buffered by tile parity) ----
    if (has_cols) {
      for (int e2 = et; e2 < BN; e2 += 32 * EW) {
        const int et_ = e2;
        const int col = n0 + et_;
        float bv = 0.f;
        if (args.bias && col < args.N) {
          if (args.bias_f32) bv = __ldg((const float*)args.bias + col);
          else {
            uint32_t u = __ldg((const uint16_t*)args.bias + col);
            bv = args.in_bf16 ? __uint_as_float(u << 16) : __half2float(__ushort_as_half((unsigned short)u));
          }
        }
        s_bias[buf * 256 + et_] = bv;
        if (ESZ == 1) {
          float sw = 1.f;
          int rs = 0;
          if (col < args.N) {
            sw = args.q_per_channel ? __ldg(args.q_sw + col) : __ldg(args.q_sw);
            rs = args.q_rowsum ? __ldg(args.q_rowsum + col) : 0;
          }
          s_qsw[buf * 256 + et_] = sw;
          s_qrs[buf * 256 + et_] = rs;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
    }
    // ---- prefetch the first chunk of the auxiliary input (next chunks: one ahead) ----
    const bool aux_fast = aux_in && aux_vec_ok && row_ok && (cbase + COLS <= args.N);
    const uint4* aux_row = reinterpret_cast<const uint4*>(
        (const uint16_t*)args.aux + (long long)b * args.strideAux + (long long)row * args.ldaux + cbase);
    uint4 auxn[4];
    if (aux_fast) {
#pragma unroll
      for (int j = 0; j < 4; j++) auxn[j] = __ldg(aux_row + j);
    }
    if (!mbar_wait(tfull, tfull_phase, abort_flag, args.status, ST_GEMM_TIMEOUT, 4)) return false;
    tc_fence_after();
    const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + half * COLS;
    // The chunk loop is deliberately not unrolled: the body is large and eight warps
    // run it; keeping one copy keeps it resident in the instruction cache.
#pragma unroll 1
    for (int c = 0; c < NCH; c++) {
      uint32_t rr[32];
      tmem_ld32(taddr + c * 32, rr);
      uint4 auxc[4];
      if (aux_fast) {
#pragma unroll
        for (int j = 0; j < 4; j++) auxc[j] = auxn[j];
        if (c + 1 < NCH) {
#pragma unroll
          for (int j = 0; j < 4; j++) auxn[j] = __ldg(aux_row + (c + 1) * 4 + j);
        }
      }
      tmem_ld_wait();
      const int col0 = cbase + c * 32;
      if (col0 >= args.N || !row_ok) continue;
      const int sc = buf * 256 + half * COLS + c * 32;  // index into the per-column arrays
      float v[32];
      if (ESZ == 1) {
#pragma unroll
        for (int j = 0; j < 32; j++)
          v[j] = q_sx * s_qsw[sc + j] * (float)((int)rr[j] - q_zx * s_qrs[sc + j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(rr[j]) * args.alpha;
      }
      if (args.bias) {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] += s_bias[sc + j];
      }
      const bool full_cols = col0 + 32 <= args.N;
      // ---- auxiliary tensor ----
      if (args.aux_mode == AUX_STORE_PRE) {
        uint16_t* ap = (uint16_t*)args.aux + (long long)b * args.strideAux + (long long)row * args.ldaux + col0;
        if (full_cols && aux_vec_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack16x(v[j], v[j + 1], args.in_bf16); o.y = pack16x(v[j + 2], v[j + 3], args.in_bf16);
            o.z = pack16x(v[j + 4], v[j + 5], args.in_bf16); o.w = pack16x(v[j + 6], v[j + 7], args.in_bf16);
            *reinterpret_cast<uint4*>(ap + j) = o;
          }
        } else {
          for (int j = 0; j < 32; j++)
            if (col0 + j < args.N) {
              if (args.in_bf16) ((__nv_bfloat16*)ap)[j] = __float2bfloat16_rn(v[j]);
              else ((__half*)ap)[j] = __float2half_rn(v[j]);
            }
        }
      }
      switch (args.act) {
        case ACT_RELU:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
          break;
        case ACT_GELU_TANH:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = gelu_tanh_f(v[j]);
          break;
        case ACT_GELU_ERF:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = gelu_erf_f(v[j]);
          break;
        default: break;
      }
      if (aux_in) {
        float a[32];
        if (aux_fast) {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint4 u = auxc[j];
            float2 f;
            f = unpack16(u.x, args.in_bf16); a[j * 8] = f.x; a[j * 8 + 1] = f.y;
            f = unpack16(u.y, args.in_bf16); a[j * 8 + 2] = f.x; a[j * 8 + 3] = f.y;
            f = unpack16(u.z, args.in_bf16); a[j * 8 + 4] = f.x; a[j * 8 + 5] = f.y;
            f = unpack16(u.w, args.in_bf16); a[j * 8 + 6] = f.x; a[j * 8 + 7] = f.y;
          }
        } else {
          const uint16_t* ap = (const uint16_t*)args.aux + (long long)b * args.strideAux + (long long)row * args.ldaux + col0;
          for (int j = 0; j < 32; j++) {
            a[j] = 0.f;
            if (col0 + j < args.N)
              a[j] = args.in_bf16 ? __bfloat162float(((const __nv_bfloat16*)ap)[j])
                                  : __half2float(((const __half*)ap)[j]);
          }
        }
        switch (args.aux_mode) {
          case AUX_ADD:
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] += a[j];
            break;
          case AUX_MUL_DGELU_TANH:
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= dgelu_tanh_f(a[j]);
            break;
          case AUX_MUL_DRELU:
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = a[j] > 0.f ? v[j] : 0.f;
            break;
          case AUX_MUL_DGELU_ERF:
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= dgelu_erf_f(a[j]);
            break;
          default: break;
        }
      }
      // ---- store ----
      if (args.out_kind == OUT_F32) {
        float* cp = (float*)args.C + (long long)b * args.strideC + (long long)row * args.ldc + col0;
        const bool v4 = full_cols && ((args.ldc & 3) == 0) && ((args.strideC & 3) == 0) &&
                        (((uintptr_t)args.C & 15) == 0);
        if (v4) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            if (args.beta) {
              float4 old = *reinterpret_cast<const float4*>(cp + j);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(cp + j) = o;
          }
        } else {
          for (int j = 0; j < 32; j++)
            if (col0 + j < args.N) cp[j] = args.beta ? cp[j] + v[j] : v[j];
        }
      } else {
        uint16_t* cp = (uint16_t*)args.C + (long long)b * args.strideC + (long long)row * args.ldc + col0;
        const bool bf = args.out_kind == OUT_BF16;
        if (full_cols && vec_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (args.beta) {
              uint4 u = *reinterpret_cast<const uint4*>(cp + j);
              float2 f;
              f = unpack16(u.x, bf); v[j] += f.x; v[j + 1] += f.y;
              f = unpack16(u.y, bf); v[j + 2] += f.x; v[j + 3] += f.y;
              f = unpack16(u.z, bf); v[j + 4] += f.x; v[j + 5] += f.y;
              f = unpack16(u.w, bf); v[j + 6] += f.x; v[j + 7] += f.y;
            }
            uint4 o;
            o.x = pack16x(v[j], v[j + 1], bf); o.y = pack16x(v[j + 2], v[j + 3], bf);
            o.z = pack16x(v[j + 4], v[j + 5], bf); o.w = pack16x(v[j + 6], v[j + 7], bf);
            *reinterpret_cast<uint4*>(cp + j) = o;
          }
        } else {
          for (int j = 0; j < 32; j++)
            if (col0 + j < args.N) {
              float x = v[j];
              if (bf) {
                if (args.beta) x += __bfloat162float(((__nv_bfloat16*)cp)[j]);
                ((__nv_bfloat16*)cp)[j] = __float2bfloat16_rn(x);
              } else {
                if (args.beta) x += __half2float(((__half*)cp)[j]);
                ((__half*)cp)[j] = __float2half_rn(x);
              }
            }
        }
      }
    }
  return true;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr)
               : "memory");
  return v;
}

// Per-warp staging state of the TMA epilogue: two 2 KB buffers (32 rows x 32 sixteen-bit
// columns, 64-byte swizzle), one mbarrier per buffer for auxiliary loads, their parities.
struct EpiStage {
  uint8_t* buf;
  uint64_t* bar;
  uint32_t phase;
};

// Epilogue through shared memory for 16-bit outputs.  A thread owns one accumulator row, so
// direct stores would touch 32 different rows per instruction (16-byte pieces of 32 lines);
// here every warp writes its 32 x 32 chunk into a swizzled staging buffer and one TMA store
// moves it out as whole lines, clipped at the matrix edge by the tensor map.  An auxiliary
// input (residual, saved pre-activation) arrives the same way, one chunk ahead, and the
// result overwrites it in place.  With a second output (saved pre-activation) buffer 0 holds
// the result and buffer 1 the pre-activation.
template <int BN, int EW>
__device__ __forceinline__ bool epilogue_tile_tma(const GemmArgs& args, const EpiCtx& cx, EpiStage& st,
                                                  const CUtensorMap* tmC, const CUtensorMap* tmX, int buf, int b,
                                                  int m0, int n0, uint32_t tmem_acc, uint64_t* tfull,
                                                  uint32_t tfull_phase, volatile int* abort_flag) {
  constexpr int COLS = BN / (EW / 4);
  constexpr int NCH = COLS / 32;
  static_assert(NCH % 2 == 0, "chunks alternate between two staging buffers");
  const int q = cx.q, half = cx.half, et = cx.et, lane = cx.lane;
  float* s_bias = cx.s_bias;
  const int mrow0 = m0 + q * 32;
  const int cbase = n0 + half * COLS;
  const bool live = mrow0 < args.M;  // warp-uniform
  const bool aux_in = cx.aux_in;
  const bool two_out = args.aux_mode == AUX_STORE_PRE;
  const int out_bf = args.out_kind == OUT_BF16;
  if (args.bias) {
    for (int e2 = et; e2 < BN; e2 += 32 * EW) {
      const int col = n0 + e2;
      float bv = 0.f;
      if (col < args.N) {
        if (args.bias_f32) bv = __ldg((const float*)args.bias + col);
        else {
          uint32_t u = __ldg((const uint16_t*)args.bias + col);
          bv = args.in_bf16 ? __uint_as_float(u << 16) : __half2float(__ushort_as_half((unsigned short)u));
        }
      }
      s_bias[buf * 256 + e2] = bv;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
  }
  const uint32_t sb0 = smem_u32(st.buf);
  const uint32_t myrow = (uint32_t)lane * 64u;
  const uint32_t swz = ((uint32_t)lane >> 1) & 3u;
  if (aux_in && live && cbase < args.N && lane == 0) {
    tma_store_wait_read<0>();  // the buffer's last store has been read out
    mbar_expect_tx(&st.bar[0], 2048);
    tma_load_3d(st.buf, tmX, &st.bar[0], cbase, mrow0, b);
  }
  if (!mbar_wait(tfull, tfull_phase, abort_flag, args.status, ST_GEMM_TIMEOUT, 4)) return false;
  tc_fence_after();
  const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + half * COLS;
#pragma unroll 1
  for (int c = 0; c < NCH; c++) {
    uint32_t rr[32];
    tmem_ld32(taddr + c * 32, rr);
    tmem_ld_wait();
    const int col0 = cbase + c * 32;
    if (!live || col0 >= args.N) continue;
    const int sc = buf * 256 + half * COLS + c * 32;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = __uint_as_float(rr[j]) * args.alpha;
    if (args.bias) {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] += s_bias[sc + j];
    }
    if (args.out_kind == OUT_F32) {
      // 32 fp32 columns are two 64-byte-wide boxes: columns 0-15 in buffer 0, 16-31 in buffer 1
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
#pragma unroll
      for (int hb = 0; hb < 2; hb++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 o;
          o.x = __float_as_uint(v[hb * 16 + j * 4]); o.y = __float_as_uint(v[hb * 16 + j * 4 + 1]);
          o.z = __float_as_uint(v[hb * 16 + j * 4 + 2]); o.w = __float_as_uint(v[hb * 16 + j * 4 + 3]);
          st_shared_v4(sb0 + hb * 2048 + myrow + (((uint32_t)j ^ swz) << 4), o);
        }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(tmC, st.buf, col0, mrow0, b);
        if (col0 + 16 < args.N) tma_store_3d(tmC, st.buf + 2048, col0 + 16, mrow0, b);
        tma_store_commit();
      }
      continue;
    }
    const int bi = c & 1;
    const uint32_t sbc = sb0 + bi * 2048;
    // second output: the pre-activation is packed now and written after the activation has
    // been computed, so that the wait for the previous chunk's stores overlaps that arithmetic
    uint4 pre_pk[4];
    if (two_out) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        pre_pk[j].x = pack16x(v[j * 8], v[j * 8 + 1], args.in_bf16);
        pre_pk[j].y = pack16x(v[j * 8 + 2], v[j * 8 + 3], args.in_bf16);
        pre_pk[j].z = pack16x(v[j * 8 + 4], v[j * 8 + 5], args.in_bf16);
        pre_pk[j].w = pack16x(v[j * 8 + 6], v[j * 8 + 7], args.in_bf16);
      }
    }
    switch (args.act) {
      case ACT_RELU:
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
        break;
      case ACT_GELU_TANH:
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = gelu_tanh_f(v[j]);
        break;
      case ACT_GELU_ERF:
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = gelu_erf_f(v[j]);
        break;
      default: break;
    }
    if (two_out) {
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 4; j++) st_shared_v4(sb0 + 2048 + myrow + (((uint32_t)j ^ swz) << 4), pre_pk[j]);
    }
    if (aux_in) {
      if (c + 1 < NCH && col0 + 32 < args.N && lane == 0) {
        tma_store_wait_read<0>();
        mbar_expect_tx(&st.bar[bi ^ 1], 2048);
        tma_load_3d(st.buf + (bi ^ 1) * 2048, tmX, &st.bar[bi ^ 1], col0 + 32, mrow0, b);
      }
      if (!mbar_wait(&st.bar[bi], (st.phase >> bi) & 1u, abort_flag, args.status, ST_GEMM_TIMEOUT, 5)) return false;
      st.phase ^= 1u << bi;
      float a[32];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint4 u = ld_shared_v4(sbc + myrow + (((uint32_t)j ^ swz) << 4));
        float2 f;
        f = unpack16(u.x, args.in_bf16); a[j * 8] = f.x; a[j * 8 + 1] = f.y;
        f = unpack16(u.y, args.in_bf16); a[j * 8 + 2] = f.x; a[j * 8 + 3] = f.y;
        f = unpack16(u.z, args.in_bf16); a[j * 8 + 4] = f.x; a[j * 8 + 5] = f.y;
        f = unpack16(u.w, args.in_bf16); a[j * 8 + 6] = f.x; a[j * 8 + 7] = f.y;
      }
      switch (args.aux_mode) {
        case AUX_ADD:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] += a[j];
          break;
        case AUX_MUL_DGELU_TANH:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= dgelu_tanh_f(a[j]);
          break;
        case AUX_MUL_DRELU:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = a[j] > 0.f ? v[j] : 0.f;
          break;
        case AUX_MUL_DGELU_ERF:
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= dgelu_erf_f(a[j]);
          break;
        default: break;
      }
    } else if (!two_out) {
      if (lane == 0) tma_store_wait_read<1>();  // the store from two chunks ago used this buffer
      __syncwarp();
    }
    const uint32_t so = two_out ? sb0 : sbc;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint4 o;
      o.x = pack16x(v[j * 8], v[j * 8 + 1], out_bf); o.y = pack16x(v[j * 8 + 2], v[j * 8 + 3], out_bf);
      o.z = pack16x(v[j * 8 + 4], v[j * 8 + 5], out_bf); o.w = pack16x(v[j * 8 + 6], v[j * 8 + 7], out_bf);
      st_shared_v4(so + myrow + (((uint32_t)j ^ swz) << 4), o);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(tmC, two_out ? st.buf : st.buf + bi * 2048, col0, mrow0, b);
      if (two_out) tma_store_3d(tmX, st.buf + 2048, col0, mrow0, b);
      tma_store_commit();
    }
  }
  return true;
}

// ESZ: operand element size (2 = bf16/fp16, 1 = int8).  A_MN / B_MN: operand
// is MN-major.  BN: tile width.
template <int ESZ, bool A_MN, bool B_MN, int BN, int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
                    const GemmArgs args) {
  using C = Cfg<ESZ, BN>;
  using SL = SmemLayout<ESZ, C::RING_BYTES, EW>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {  // the swizzled layouts below assume this
    if (threadIdx.x == 0) set_status(args.status, ST_BAD_INDEX, 1024);
    return;
  }
  uint64_t* bars = (uint64_t*)(smem + SL::OFF_BARS);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * C::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  uint64_t* aux_bar = bars + 32;                // [EW][2], 16-bit path
  float* s_bias = (float*)(smem + SL::OFF_COLS);   // [2][256]
  float* s_qsw = s_bias + 512;                     // [2][256]  (8-bit path only)
  int* s_qrs = (int*)(s_qsw + 512);                // [2][256]  (8-bit path only)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (args.K + C::BK - 1) / C::BK;
  const int num_tiles = args.num_m * args.num_n * args.batch * args.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], EW);  // one arrive per epilogue warp
    }
    for (int i = 0; i < 2 * EW; i++) mbar_init(&aux_bar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (args.tma_epi) {
      tma_prefetch_desc(&tmC);
      if (args.aux_mode != AUX_NONE) tma_prefetch_desc(&tmX);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Unit u = decode_unit(t, args);
        const int b = u.b;
        const int m0 = u.mb * BM, n0 = u.nb * BN;
        const int kb_end = min(num_kb, (u.s + 1) * args.kb_per);
        for (int kb = u.s * args.kb_per; kb < kb_end; kb++) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status, ST_GEMM_TIMEOUT, 1);
          if (!ok) break;
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
          const int k0 = kb * C::BK;
          const int ba = args.bcastA ? 0 : b, bb = args.bcastB ? 0 : b;
          if (!A_MN) {
            tma_load_3d(sa, &tmA, &full_bar[stage], k0, m0, ba);
          } else {
            constexpr int MN_ATOM = kSwizzleBytes / ESZ;  // elements along M per box
#pragma unroll
            for (int i = 0; i < BM / MN_ATOM; i++)
              tma_load_3d(sa + i * (C::BK * kSwizzleBytes), &tmA, &full_bar[stage], m0 + i * MN_ATOM,
                          k0, ba);
          }
          if (!B_MN) {
            tma_load_3d(sb, &tmB, &full_bar[stage], k0, n0, bb);
          } else {
            constexpr int MN_ATOM = kSwizzleBytes / ESZ;
#pragma unroll
            for (int i = 0; i < BN / MN_ATOM; i++)
              tma_load_3d(sb + i * (C::BK * kSwizzleBytes), &tmB, &full_bar[stage], n0 + i * MN_ATOM,
                          k0, bb);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before the CTA exits
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc =
        make_idesc(ESZ == 1 ? 2u : 1u, 0u, A_MN, B_MN, BM, BN);  // formats patched below
    uint32_t id = idesc;
    if (ESZ == 1) {
      id |= (1u << 7) | (1u << 10);  // signed 8-bit A and B
    } else if (args.in_bf16) {
      id |= (1u << 7) | (1u << 10);  // bf16 A and B
    }
    // One elected thread runs the whole issue loop (waits included): no per-k-block
    // reconvergence of the warp, and the compiler sees a single-thread instruction stream.
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tphase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local_tile++) {
        const int buf = local_tile & 1;
        ok = mbar_wait(&tempty_bar[buf], tphase[buf] ^ 1, abort_flag, args.status, ST_GEMM_TIMEOUT, 2);
        if (!ok) break;
        tphase[buf] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int slice = t / (num_tiles / args.splits);
        const int kb_begin = slice * args.kb_per, kb_end = min(num_kb, kb_begin + args.kb_per);
        for (int kb = kb_begin; kb < kb_end; kb++) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, args.status, ST_GEMM_TIMEOUT, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < C::BK / C::UMMA_K; k++) {
            // K-major: 8-row groups are 1024 B apart, one MMA step is 32 B along K.
            // MN-major: 64-element (128 B) chunks along MN are BK*128 B apart (LBO),
            // 8-row k groups 1024 B apart (SBO); one MMA step covers UMMA_K rows.
            const uint64_t adesc =
                A_MN ? make_smem_desc_sw128(sa + k * C::UMMA_K * kSwizzleBytes,
                                            C::BK * kSwizzleBytes, 1024)
                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc_sw128(sb + k * C::UMMA_K * kSwizzleBytes,
                                            C::BK * kSwizzleBytes, 1024)
                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            if (ESZ == 1)
              tc_mma_i8(d_tmem, adesc, bdesc, id, (kb > kb_begin) || k != 0);
            else
              tc_mma_f16(d_tmem, adesc, bdesc, id, (kb > kb_begin) || k != 0);
          }
          tc_commit(&empty_bar[stage]);
          if (kb == kb_end - 1) tc_commit(&tfull_bar[buf]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    // Two warps per TMEM lane quarter; each handles half of the tile's columns.
    // Everything that does not depend on the accumulator (bias, residual / saved
    // pre-activation) is fetched BEFORE waiting for the MMAs, so those latencies
    // overlap the main loop of the tile.
    const EpiCtx cx = make_epi_ctx<ESZ>(args, warp, lane, threadIdx.x - 64, s_bias, s_qsw, s_qrs);
    EpiStage est;
    est.buf = smem + SL::OFF_STAGING + (warp - 2) * 2 * SL::kStageBuf;
    est.bar = aux_bar + (warp - 2) * 2;
    est.phase = 0;
    uint32_t tphase[2] = {0, 0};
    int local_tile = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local_tile++) {
      const int buf = local_tile & 1;
      const Unit u = decode_unit(t, args);
      const int b = u.s * args.batch + u.b;  // slices of a split launch are stacked like batch entries
      const int m0 = u.mb * BM, n0 = u.nb * BN;
      bool done;
      if (ESZ == 2 && args.tma_epi)
        done = epilogue_tile_tma<BN, EW>(args, cx, est, &tmC, &tmX, buf, b, m0, n0, tmem_base + buf * BN,
                                         &tfull_bar[buf], tphase[buf], abort_flag);
      else
        done = epilogue_tile<ESZ, BN, EW>(args, cx, buf, b, m0, n0, tmem_base + buf * BN, &tfull_bar[buf],
                                          tphase[buf], abort_flag);
      if (!done) {
        ok = false;
        break;
      }
      tphase[buf] ^= 1;
      // accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    // shared memory must outlive the stores that read from it
    if (ESZ == 2 && args.tma_epi && lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Two-CTA variant: a cluster of two CTAs (two SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 of
// the 256 columns of B (so B crosses the L2 -> SM path once per pair instead of twice,
// and a stage is 32 KB instead of 48 KB: six stages fit), and owns 128 rows of the
// accumulator in its TMEM.  CTA 0 issues the MMAs for the pair.  Every TMA load is an
// ordinary per-CTA load; nothing is broadcast across the cluster.
// ---------------------------------------------------------------------------
constexpr uint32_t kPeerBit = 1u << 24;  // shared::cluster address bit that selects CTA 1 of a pair

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d_2sm(void* dst, const CUtensorMap* m, uint32_t bar_addr, int c0,
                                                int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"((uint64_t)m), "r"(bar_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_2sm(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (when the issuing thread's earlier MMAs retire) on the barrier at a shared::cluster address
__device__ __forceinline__ void tc_commit_2sm(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}

struct Cfg2 {
  static constexpr int BN = 256;                 // columns of the pair tile (each CTA stages 128 of them)
  static constexpr int BK = 64;
  static constexpr int UMMA_K = 16;
  static constexpr int A_BYTES = 128 * kSwizzleBytes;
  static constexpr int B_BYTES = 128 * kSwizzleBytes;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TMEM_COLS = 512;
};

template <bool A_MN, bool B_MN, int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
                         const GemmArgs args) {
  using C = Cfg2;
  using SL = SmemLayout<2, C::RING_BYTES, EW>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) set_status(args.status, ST_BAD_INDEX, 1024);
    return;
  }
  uint64_t* bars = (uint64_t*)(smem + SL::OFF_BARS);
  uint64_t* full_bar = bars;                   // [STAGES]  used in CTA 0
  uint64_t* empty_bar = bars + C::STAGES;      // [STAGES]  per CTA
  uint64_t* tfull_bar = bars + 2 * C::STAGES;  // [2]       per CTA
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]       used in CTA 0
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  uint64_t* aux_bar = bars + 32;               // [EW][2]   per CTA
  float* s_bias = (float*)(smem + SL::OFF_COLS);
  float* s_qsw = s_bias;   // 8-bit constants are not used by this kernel
  int* s_qrs = (int*)s_bias;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();      // 0: leader (issues the MMAs), 1: peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (args.K + C::BK - 1) / C::BK;
  // num_m / num_n count 256 x 256 pair tiles here
  const int num_tiles = args.num_m * args.num_n * args.batch * args.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 2 * EW);  // the epilogue warps of both CTAs
    }
    for (int i = 0; i < 2 * EW; i++) mbar_init(&aux_bar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (args.tma_epi) {
      tma_prefetch_desc(&tmC);
      if (args.aux_mode != AUX_NONE) tma_prefetch_desc(&tmX);
    }
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, C::TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised before anyone touches the peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const Unit u = decode_unit(t, args);
        const int b = u.b;
        const int m0 = u.mb * 256 + (int)cta * 128;   // this CTA's rows of A
        const int n0 = u.nb * 256 + (int)cta * 128;   // this CTA's columns of B
        const int kb_end = min(num_kb, (u.s + 1) * args.kb_per);
        for (int kb = u.s * args.kb_per; kb < kb_end; kb++) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status, ST_GEMM_TIMEOUT, 11);
          if (!ok) break;
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          // bytes of both CTAs land on the leader's barrier
          const uint32_t fb = smem_u32(&full_bar[stage]) & ~kPeerBit;
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * C::STAGE_BYTES);
          const int k0 = kb * C::BK;
          const int ba = args.bcastA ? 0 : b, bb = args.bcastB ? 0 : b;
          if (!A_MN) {
            tma_load_3d_2sm(sa, &tmA, fb, k0, m0, ba);
          } else {
#pragma unroll
            for (int i = 0; i < 2; i++) tma_load_3d_2sm(sa + i * (C::BK * kSwizzleBytes), &tmA, fb, m0 + i * 64, k0, ba);
          }
          if (!B_MN) {
            tma_load_3d_2sm(sb, &tmB, fb, k0, n0, bb);
          } else {
#pragma unroll
            for (int i = 0; i < 2; i++) tma_load_3d_2sm(sb + i * (C::BK * kSwizzleBytes), &tmB, fb, n0 + i * 64, k0, bb);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (cta == 0 && elect_one()) {
      uint32_t id = make_idesc(1u, args.in_bf16 ? 1u : 0u, A_MN, B_MN, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tphase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, local_tile++) {
        const int buf = local_tile & 1;
        ok = mbar_wait(&tempty_bar[buf], tphase[buf] ^ 1, abort_flag, args.status, ST_GEMM_TIMEOUT, 12);
        if (!ok) break;
        tphase[buf] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        const int slice = t / (num_tiles / args.splits);
        const int kb_begin = slice * args.kb_per, kb_end = min(num_kb, kb_begin + args.kb_per);
        for (int kb = kb_begin; kb < kb_end; kb++) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, args.status, ST_GEMM_TIMEOUT, 13);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < C::BK / C::UMMA_K; k++) {
            const uint64_t adesc =
                A_MN ? make_smem_desc_sw128(sa + k * C::UMMA_K * kSwizzleBytes, C::BK * kSwizzleBytes, 1024)
                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc_sw128(sb + k * C::UMMA_K * kSwizzleBytes, C::BK * kSwizzleBytes, 1024)
                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_f16_2sm(d_tmem, adesc, bdesc, id, (kb > kb_begin) || k != 0);
          }
          // free the stage in both CTAs
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          tc_commit_2sm(eb);
          tc_commit_2sm(eb | kPeerBit);
          if (kb == kb_end - 1) {
            const uint32_t tb = smem_u32(&tfull_bar[buf]);
            tc_commit_2sm(tb);
            tc_commit_2sm(tb | kPeerBit);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: this CTA's 128 rows x 256 columns ----------------
    const EpiCtx cx = make_epi_ctx<2>(args, warp, lane, threadIdx.x - 64, s_bias, s_qsw, s_qrs);
    EpiStage est;
    est.buf = smem + SL::OFF_STAGING + (warp - 2) * 2 * SL::kStageBuf;
    est.bar = aux_bar + (warp - 2) * 2;
    est.phase = 0;
    uint32_t tphase[2] = {0, 0};
    int local_tile = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, local_tile++) {
      const int buf = local_tile & 1;
      const Unit u = decode_unit(t, args);
      const int b = u.s * args.batch + u.b;
      const int m0 = u.mb * 256 + (int)cta * 128, n0 = u.nb * 256;
      bool done;
      if (args.tma_epi)
        done = epilogue_tile_tma<256, EW>(args, cx, est, &tmC, &tmX, buf, b, m0, n0, tmem_base + buf * 256,
                                          &tfull_bar[buf], tphase[buf], abort_flag);
      else
        done = epilogue_tile<2, 256, EW>(args, cx, buf, b, m0, n0, tmem_base + buf * 256, &tfull_bar[buf],
                                         tphase[buf], abort_flag);
      if (!done) {
        ok = false;
        break;
      }
      tphase[buf] ^= 1;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(smem_u32(&tempty_bar[buf]) & ~kPeerBit);
    }
    if (args.tma_epi && lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves while the other may still use its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// SIMT fallback for fp32 / fp64 operands (exact-precision parity paths)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                                 int M, int N, int K, int transA, int transB, long long lda,
                                 long long ldb, long long ldc, long long sA, long long sB,
                                 long long sC, T alpha, int beta) {
  constexpr int TS = 64, KS = 16;
  __shared__ T As[KS][TS + 1];
  __shared__ T Bs[KS][TS + 1];
  const int b = blockIdx.z;
  A += (long long)b * sA;
  B += (long long)b * sB;
  C += (long long)b * sC;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);
  for (int k0 = 0; k0 < K; k0 += KS) {
    for (int i = threadIdx.x; i < TS * KS; i += 256) {
      int kk, mm;
      if (transA) { mm = i % TS; kk = i / TS; } else { kk = i % KS; mm = i / KS; }
      int gm = m0 + mm, gk = k0 + kk;
      T v = T(0);
      if (gm < M && gk < K) v = transA ? A[(long long)gk * lda + gm] : A[(long long)gm * lda + gk];
      As[kk][mm] = v;
    }
    for (int i = threadIdx.x; i < TS * KS; i += 256) {
      int kk, nn;
      if (transB) { kk = i % KS; nn = i / KS; } else { nn = i % TS; kk = i / TS; }
      int gn = n0 + nn, gk = k0 + kk;
      T v = T(0);
      if (gn < N && gk < K) v = transB ? B[(long long)gn * ldb + gk] : B[(long long)gk * ldb + gn];
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KS; kk++) {
      T a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * bb[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      T* p = C + (long long)gm * ldc + gn;
      T v = alpha * acc[i][j];
      *p = beta ? (*p + v) : v;
    }
  }
}

// Register-tiled SIMT GEMM for fp32 / fp64: 256 threads as a 16 x 16 grid, each thread owns
// TM x TN outputs laid out in 16-byte groups (VEC elements) that interleave across the
// threads, so that every shared-memory read is one conflict-free 128-bit load and a row of
// 16 threads writes 256 contiguous bytes of C.  Tiles are staged k-major in two shared-memory
// buffers; the next tile travels global -> registers while the current one is multiplied.
template <typename T, int TM, int TN, int BK>
__global__ void __launch_bounds__(256, 2)
gemm_simt_tiled_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int M,
                       int N, int K, int transA, int transB, long long lda, long long ldb,
                       long long ldc, long long sA, long long sB, long long sC, T alpha, int beta) {
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int BM = 16 * TM, BN = 16 * TN, PAD = VEC;
  constexpr int LA = BM * BK / 256, LB = BN * BK / 256;
  static_assert(TM % VEC == 0 && TN % VEC == 0, "thread tile must be whole 16-byte groups");
  static_assert((BM * BK) % 256 == 0 && (BN * BK) % 256 == 0, "tile must divide among 256 threads");
  struct alignas(16) Vec { T v[VEC]; };
  __shared__ __align__(16) T As[2][BK][BM + PAD];
  __shared__ __align__(16) T Bs[2][BK][BN + PAD];

  const int b = blockIdx.z;
  A += (long long)b * sA;
  B += (long long)b * sB;
  C += (long long)b * sC;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = T(0);
  T ra[LA], rb[LB];

  auto load_global = [&](int k0) {
#pragma unroll
    for (int r = 0; r < LA; r++) {
      const int i = tid + r * 256;
      int kk, mm;
      if (transA) { mm = i % BM; kk = i / BM; } else { kk = i % BK; mm = i / BK; }
      const int gm = m0 + mm, gk = k0 + kk;
      T v = T(0);
      if (gm < M && gk < K) v = transA ? A[(long long)gk * lda + gm] : A[(long long)gm * lda + gk];
      ra[r] = v;
    }
#pragma unroll
    for (int r = 0; r < LB; r++) {
      const int i = tid + r * 256;
      int kk, nn;
      if (transB) { kk = i % BK; nn = i / BK; } else { nn = i % BN; kk = i / BN; }
      const int gn = n0 + nn, gk = k0 + kk;
      T v = T(0);
      if (gn < N && gk < K) v = transB ? B[(long long)gn * ldb + gk] : B[(long long)gk * ldb + gn];
      rb[r] = v;
    }
  };
  auto store_shared = [&](int buf) {
#pragma unroll
    for (int r = 0; r < LA; r++) {
      const int i = tid + r * 256;
      int kk, mm;
      if (transA) { mm = i % BM; kk = i / BM; } else { kk = i % BK; mm = i / BK; }
      As[buf][kk][mm] = ra[r];
    }
#pragma unroll
    for (int r = 0; r < LB; r++) {
      const int i = tid + r * 256;
      int kk, nn;
      if (transB) { kk = i % BK; nn = i / BK; } else { nn = i % BN; kk = i / BN; }
      Bs[buf][kk][nn] = rb[r];
    }
  };

  const int nk = (K + BK - 1) / BK;
  if (nk > 0) {
    load_global(0);
    store_shared(0);
  }
  __syncthreads();
  for (int t = 0; t < nk; t++) {
    const int buf = t & 1;
    if (t + 1 < nk) load_global((t + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      T a[TM], bb[TN];
#pragma unroll
      for (int g = 0; g < TM / VEC; g++) {
        const Vec va = *reinterpret_cast<const Vec*>(&As[buf][kk][g * 16 * VEC + ty * VEC]);
#pragma unroll
        for (int v = 0; v < VEC; v++) a[g * VEC + v] = va.v[v];
      }
#pragma unroll
      for (int h = 0; h < TN / VEC; h++) {
        const Vec vb = *reinterpret_cast<const Vec*>(&Bs[buf][kk][h * 16 * VEC + tx * VEC]);
#pragma unroll
        for (int v = 0; v < VEC; v++) bb[h * VEC + v] = vb.v[v];
      }
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] += a[i] * bb[j];
    }
    if (t + 1 < nk) store_shared(buf ^ 1);
    __syncthreads();   // buf^1 is complete, and nobody still reads buf when it is refilled next
  }

  const bool vec_ok = (reinterpret_cast<unsigned long long>(C) % 16 == 0) && (ldc % VEC == 0);
#pragma unroll
  for (int g = 0; g < TM / VEC; g++) {
#pragma unroll
    for (int vi = 0; vi < VEC; vi++) {
      const int gm = m0 + g * 16 * VEC + ty * VEC + vi;
      if (gm >= M) continue;
      const int i = g * VEC + vi;
#pragma unroll
      for (int h = 0; h < TN / VEC; h++) {
        const int gn = n0 + h * 16 * VEC + tx * VEC;
        if (gn >= N) continue;
        T* p = C + (long long)gm * ldc + gn;
        if (vec_ok && gn + VEC <= N) {
          Vec o;
          if (beta) o = *reinterpret_cast<const Vec*>(p);
#pragma unroll
          for (int v = 0; v < VEC; v++) {
            const T r = alpha * acc[i][h * VEC + v];
            o.v[v] = beta ? (o.v[v] + r) : r;
          }
          *reinterpret_cast<Vec*>(p) = o;
        } else {
#pragma unroll
          for (int v = 0; v < VEC; v++) {
            if (gn + v >= N) continue;
            const T r = alpha * acc[i][h * VEC + v];
            p[v] = beta ? (p[v] + r) : r;
          }
        }
      }
    }
  }
}

int g_simt_tiled = 1;   // 0 selects the plain 64 x 64 kernel above

template <typename T, int TM, int TN, int BK>
void launch_simt_tiled(const void* A, const void* B, void* C, int M, int N, int K, int batch,
                       int transA, int transB, long long lda, long long ldb, long long ldc,
                       long long sA, long long sB, long long sC, double alpha, int beta,
                       cudaStream_t stream) {
  dim3 grid((N + 16 * TN - 1) / (16 * TN), (M + 16 * TM - 1) / (16 * TM), batch);
  gemm_simt_tiled_kernel<T, TM, TN, BK><<<grid, 256, 0, stream>>>(
      (const T*)A, (const T*)B, (T*)C, M, N, K, transA, transB, lda, ldb, ldc, sA, sB, sC, (T)alpha,
      beta);
}

int g_epi_warps = 8;

struct TMaps {
  CUtensorMap a, b, c, x;  // operands, output, auxiliary tensor
};

template <int ESZ, bool A_MN, bool B_MN, int BN, int EW>
int launch_tc_ew(const TMaps& tm, const GemmArgs& args, int num_sms, cudaStream_t stream) {
  using C = Cfg<ESZ, BN>;
  using SL = SmemLayout<ESZ, C::RING_BYTES, EW>;
  auto kern = gemm_tcgen05_kernel<ESZ, A_MN, B_MN, BN, EW>;
  static bool configured = false;
  if (!configured) {
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL::BYTES));
    configured = true;
  }
  int tiles = args.num_m * args.num_n * args.batch * args.splits;
  int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, 64 + 32 * EW, SL::BYTES, stream>>>(tm.a, tm.b, tm.c, tm.x, args);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <int ESZ, bool A_MN, bool B_MN, int BN>
int launch_tc(const TMaps& tm, const GemmArgs& args, int num_sms, cudaStream_t stream) {
  if (g_epi_warps == 4) return launch_tc_ew<ESZ, A_MN, B_MN, BN, 4>(tm, args, num_sms, stream);
  return launch_tc_ew<ESZ, A_MN, B_MN, BN, 8>(tm, args, num_sms, stream);
}

template <int ESZ, int BN>
int dispatch_major(bool a_mn, bool b_mn, const TMaps& tm, const GemmArgs& args, int num_sms,
                   cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_tc<ESZ, false, false, BN>(tm, args, num_sms, stream);
  if (ESZ == 2) {
    if (!a_mn && b_mn) return launch_tc<2, false, true, BN>(tm, args, num_sms, stream);
    if (a_mn && !b_mn) return launch_tc<2, true, false, BN>(tm, args, num_sms, stream);
    return launch_tc<2, true, true, BN>(tm, args, num_sms, stream);
  }
  gbh::set_error("int8 GEMM supports only A (M,K) row-major with B (N,K) row-major");
  return gbh::E_BAD_ARG;
}


int g_use_2cta = 1;

template <bool A_MN, bool B_MN>
int launch_2cta(const TMaps& tm, const GemmArgs& args, int num_sms, cudaStream_t stream) {
  using SL = SmemLayout<2, Cfg2::RING_BYTES, 8>;
  auto kern = gemm_tcgen05_2cta_kernel<A_MN, B_MN, 8>;
  static bool configured = false;
  if (!configured) {
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL::BYTES));
    configured = true;
  }
  int tiles = args.num_m * args.num_n * args.batch * args.splits;
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(64 + 32 * 8);
  cfg.dynamicSmemBytes = SL::BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tm.a, tm.b, tm.c, tm.x, args));
  return gbh::E_OK;
}

// Sums the K slices of a split launch in slice order and writes the result in the
// caller's type: C = (beta ? C : 0) + sum_s ws[s].
template <typename TO>
__global__ void splitk_finish_kernel(const float* __restrict__ ws, TO* __restrict__ C, int M, int N, int batch,
                                     int splits, long long ldc, long long strideC, int beta) {
  const long long per = (long long)M * N;
  const long long total = per * batch;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total;
       i += (long long)gridDim.x * blockDim.x * 4) {
    // N is a multiple of 4 here, so the four elements share a row
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; s++) {
      const float4 v = *reinterpret_cast<const float4*>(ws + s * total + i);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    long long b, m, n;
    if (total <= 0x7fffffffLL) {          // 32-bit index arithmetic: the 64-bit divisions cost more than the sums
      const unsigned ui = (unsigned)i, uper = (unsigned)per, uN = (unsigned)N;
      const unsigned ub = ui / uper, ur = ui - ub * uper, um = ur / uN;
      b = ub; m = um; n = ur - um * uN;
    } else {
      b = i / per;
      const long long r = i - b * per;
      m = r / N;
      n = r - m * N;
    }
    TO* c = C + b * strideC + m * ldc + n;
    if (sizeof(TO) == 2 && (((uintptr_t)c & 7) == 0)) {
      // four 16-bit results as one 8-byte access
      uint2 raw;
      if (beta) {
        raw = *reinterpret_cast<const uint2*>(c);
        const TO* e = reinterpret_cast<const TO*>(&raw);
        a.x += (float)e[0]; a.y += (float)e[1]; a.z += (float)e[2]; a.w += (float)e[3];
      }
      TO o[4] = {(TO)a.x, (TO)a.y, (TO)a.z, (TO)a.w};
      *reinterpret_cast<uint2*>(c) = *reinterpret_cast<const uint2*>(o);
    } else {
      if (beta) { a.x += (float)c[0]; a.y += (float)c[1]; a.z += (float)c[2]; a.w += (float)c[3]; }
      c[0] = (TO)a.x; c[1] = (TO)a.y; c[2] = (TO)a.z; c[3] = (TO)a.w;
    }
  }
}

int g_splitk = 1;

// Number of K slices for a launch with `tiles` output tiles on `slots` concurrently running
// CTAs (or CTA pairs): the count that fills whole waves best, with a small bias towards
// fewer slices (less workspace traffic).  1 = do not split.
int pick_splits(long long tiles, int slots, int num_kb, long long slice_bytes, long long workspace_bytes) {
  if (tiles * 4 > (long long)slots * 3 || num_kb < 32) return 1;
  int best = 1;
  double best_score = (double)tiles / slots - 0.01;
  for (int s = 2; s <= 16; s++) {
    if (num_kb / s < 16 || slice_bytes * s > workspace_bytes) break;
    const long long units = tiles * s;
    const long long waves = (units + slots - 1) / slots;
    const double score = (double)units / (double)(waves * slots) - 0.01 * s;
    if (score > best_score + 1e-9) { best_score = score; best = s; }
  }
  return best;
}

int g_num_sms = 0;
int g_group_m = 8;
int g_tma_epi = 1;

// Builds the two tensor maps and launches.  esz: 2 (bf16/fp16) or 1 (int8).
int gemm_tc(int esz, const void* A, const void* B, GemmArgs& args, int transA, int transB,
            long long lda, long long ldb, long long sA, long long sB, int force_bn,
            cudaStream_t stream, void* workspace = nullptr, long long workspace_bytes = 0) {
  if (g_num_sms == 0) {
    int dev = 0;
    GB_CUDA_OK(cudaGetDevice(&dev));
    GB_CUDA_OK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const bool a_mn = transA != 0;  // stored K x M
  const bool b_mn = transB == 0;  // stored K x N
  const int M = args.M, N = args.N, K = args.K, batch = args.batch;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) {
    gbh::set_error("gemm: empty problem M=%d N=%d K=%d batch=%d", M, N, K, batch);
    return gbh::E_BAD_ARG;
  }
  const int atom = kSwizzleBytes / esz;  // elements in one 128-byte row
  // choose tile width: the narrow tile when the wide one cannot fill the GPU
  int bn = 256;
  {
    long long tiles256 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256) * batch;
    if (N <= 128 || tiles256 < g_num_sms) bn = 128;
  }
  if (force_bn == 128 || force_bn == 256) bn = force_bn;
  // two-CTA 256 x 256 tiles when they fill at least four fifths of the SM pairs (measured at 2048^3: 64 pair
  // tiles on 74 pairs beat 128 one-CTA tiles on 148 SMs by 8 %); force_bn == 512 forces them
  bool use2 = false;
  if (esz == 2) {
    long long pair_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256) * batch;
    // measured: the pair kernel wins when the main loop dominates (long K, or a plain
    // epilogue); with short K and a heavy epilogue the one-CTA kernel is slightly ahead
    const bool light = args.act == ACT_NONE && args.aux_mode == AUX_NONE;
    use2 = force_bn == 512 || (force_bn == 0 && g_use_2cta && pair_tiles * 5 >= (long long)(g_num_sms / 2) * 4 && M >= 256 &&
                               N >= 256 && (K >= 1536 || light));
  }
  // Split-K: a product with few output tiles and a long K is cut into K slices that run as
  // separate work units into an fp32 workspace; a second kernel adds them in slice order.
  args.splits = 1;
  args.kb_per = (K + atom - 1) / atom;
  int splits = 1;
  const bool plain = args.bias == nullptr && args.act == ACT_NONE && args.aux_mode == AUX_NONE;
  const bool big = 2.0 * M * N * (double)K * batch >= 8e9;  // below this the second launch costs more than it saves
  if (esz == 2 && g_splitk && force_bn == 0 && plain && big && workspace != nullptr && (N & 3) == 0 &&
      M >= 128 && N >= 128) {
    const int num_kb = (K + atom - 1) / atom;
    const long long slice_bytes = (long long)M * N * batch * 4;
    const long long t1 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256) * batch;
    const long long t2 = (long long)((M + 255) / 256) * ((N + 255) / 256) * batch;
    const bool pair_ok = g_use_2cta && M >= 256 && N >= 256;
    const int s2 = pair_ok ? pick_splits(t2, g_num_sms / 2, num_kb, slice_bytes, workspace_bytes) : 1;
    const int s1 = pick_splits(t1, g_num_sms, num_kb, slice_bytes, workspace_bytes);
    if (s2 > 1) { splits = s2; use2 = true; }
    else if (s1 > 1) { splits = s1; use2 = false; bn = 256; }
  }
  void* user_C = args.C;
  const long long user_ldc = args.ldc, user_strideC = args.strideC;
  const int user_out = args.out_kind, user_beta = args.beta;
  if (splits > 1) {
    const int num_kb = (K + atom - 1) / atom;
    args.splits = splits;
    args.kb_per = (num_kb + splits - 1) / splits;
    if ((long long)(splits - 1) * args.kb_per >= num_kb) {  // the last slice would be empty
      args.splits = splits = (num_kb + args.kb_per - 1) / args.kb_per;
    }
    args.C = workspace;
    args.ldc = N;
    args.strideC = (long long)M * N;
    args.out_kind = OUT_F32;
    args.beta = 0;
  }
  if (use2) bn = 128;   // each CTA of a pair stages 128 of the tile's 256 columns
  args.num_m = use2 ? (M + 255) / 256 : (M + BM - 1) / BM;
  args.num_n = use2 ? (N + 255) / 256 : (N + bn - 1) / bn;
  args.status = gbh::status_ptr();
  args.group_m = g_group_m;

  CUtensorMapDataType dt = esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : (args.in_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  TMaps tm;
  memset(&tm, 0, sizeof(tm));
  CUtensorMap& tmA = tm.a;
  CUtensorMap& tmB = tm.b;
  // Results of 16-bit kernels leave through shared memory and TMA stores when the output
  // (and the auxiliary tensor) can be described by a tensor map and nothing is accumulated.
  args.tma_epi = 0;
  const bool f32_out = args.out_kind == OUT_F32;
  if (esz == 2 && g_tma_epi && !args.beta && !(f32_out && (args.act != ACT_NONE || args.aux_mode != AUX_NONE))) {
    const int osz = f32_out ? 4 : 2;
    auto mappable = [&](const void* p, long long ld, long long bs) {
      return (((uintptr_t)p & 15) == 0) && (ld * osz % 16 == 0) && (bs * osz % 16 == 0);
    };
    bool ok = mappable(args.C, args.ldc, args.strideC) &&
              (args.aux_mode == AUX_NONE || mappable(args.aux, args.ldaux, args.strideAux));
    if (ok) {
      // a split launch stacks its K slices like batch entries
      const int nb = batch * args.splits;
      auto encode_out = [&](CUtensorMap* m, const void* p, long long ld, long long bs, int sz) {
        uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)nb};
        uint64_t strides[2] = {(uint64_t)ld * sz, (uint64_t)(nb > 1 ? bs : (long long)M * ld) * sz};
        uint32_t box[3] = {(uint32_t)(64 / sz), 32, 1};
        return gbh::encode_tmap(m, sz == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, p,
                                dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
      };
      int rc = encode_out(&tm.c, args.C, args.ldc, args.strideC, osz);
      if (rc) return rc;
      if (args.aux_mode != AUX_NONE) {
        rc = encode_out(&tm.x, args.aux, args.ldaux, args.strideAux, 2);
        if (rc) return rc;
      }
      args.tma_epi = 1;
    }
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a_mn) {
      dims[0] = K; dims[1] = M; dims[2] = batch;
      box[0] = atom; box[1] = BM; box[2] = 1;
    } else {
      dims[0] = M; dims[1] = K; dims[2] = batch;
      box[0] = atom; box[1] = atom; box[2] = 1;
    }
    strides[0] = (uint64_t)lda * esz;
    args.bcastA = (batch > 1 && sA == 0);
    if (batch == 1 || args.bcastA) dims[2] = 1;
    strides[1] = (uint64_t)(dims[2] > 1 ? sA : (long long)dims[1] * lda) * esz;
    int rc = gbh::encode_tmap(&tmA, dt, 3, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!b_mn) {
      dims[0] = K; dims[1] = N; dims[2] = batch;
      box[0] = atom; box[1] = bn; box[2] = 1;
    } else {
      dims[0] = N; dims[1] = K; dims[2] = batch;
      box[0] = atom; box[1] = atom; box[2] = 1;
    }
    strides[0] = (uint64_t)ldb * esz;
    args.bcastB = (batch > 1 && sB == 0);
    if (batch == 1 || args.bcastB) dims[2] = 1;
    strides[1] = (uint64_t)(dims[2] > 1 ? sB : (long long)dims[1] * ldb) * esz;
    int rc = gbh::encode_tmap(&tmB, dt, 3, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  int rc;
  if (use2) {
    if (!a_mn && !b_mn) rc = launch_2cta<false, false>(tm, args, g_num_sms, stream);
    else if (!a_mn && b_mn) rc = launch_2cta<false, true>(tm, args, g_num_sms, stream);
    else if (a_mn && !b_mn) rc = launch_2cta<true, false>(tm, args, g_num_sms, stream);
    else rc = launch_2cta<true, true>(tm, args, g_num_sms, stream);
  } else if (esz == 2) {
    if (bn == 256) rc = dispatch_major<2, 256>(a_mn, b_mn, tm, args, g_num_sms, stream);
    else rc = dispatch_major<2, 128>(a_mn, b_mn, tm, args, g_num_sms, stream);
  } else {
    if (bn == 256) rc = dispatch_major<1, 256>(a_mn, b_mn, tm, args, g_num_sms, stream);
    else rc = dispatch_major<1, 128>(a_mn, b_mn, tm, args, g_num_sms, stream);
  }
  if (rc != gbh::E_OK || splits == 1) return rc;
  {
    const long long quads = (long long)M * N * batch / 4;
    const int grid = (int)(quads + 255) / 256 < g_num_sms * 8 ? (int)((quads + 255) / 256) : g_num_sms * 8;
    const float* ws = (const float*)workspace;
    if (user_out == OUT_F32)
      splitk_finish_kernel<float><<<grid, 256, 0, stream>>>(ws, (float*)user_C, M, N, batch, splits, user_ldc,
                                                            user_strideC, user_beta);
    else if (user_out == OUT_BF16)
      splitk_finish_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(ws, (__nv_bfloat16*)user_C, M, N, batch,
                                                                    splits, user_ldc, user_strideC, user_beta);
    else
      splitk_finish_kernel<__half><<<grid, 256, 0, stream>>>(ws, (__half*)user_C, M, N, batch, splits,
                                                             user_ldc, user_strideC, user_beta);
    GB_CUDA_OK(cudaGetLastError());
  }
  return gbh::E_OK;
}

}  // namespace

// Tuning knobs: epilogue warps (4 or 8) and rasterisation group height (row blocks).
GB_EXPORT int gb_gemm_tune(int epi_warps, int group_m) {
  if (epi_warps == 4 || epi_warps == 8) g_epi_warps = epi_warps;
  if (group_m >= 1) g_group_m = group_m;
  return 0;
}
// Selects the register-tiled fp32 / fp64 kernel (1, the default) or the plain 64 x 64 one (0).
GB_EXPORT int gb_gemm_simt_tiled(int on) {
  g_simt_tiled = on;
  return 0;
}
// Enables (1) or disables (0) the automatic choice of the two-CTA kernel.
GB_EXPORT int gb_gemm_use_2cta(int on) {
  g_use_2cta = on;
  return 0;
}
// Enables (1) or disables (0) split-K for products with few output tiles.
GB_EXPORT int gb_gemm_splitk(int on) {
  g_splitk = on;
  return 0;
}
// Enables (1) or disables (0) the shared-memory + TMA-store epilogue of the 16-bit kernels.
GB_EXPORT int gb_gemm_tma_epilogue(int on) {
  g_tma_epi = on;
  return 0;
}

// dtype codes shared with the Python side
enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3, DT_I8 = 4 };

// 16-bit tensor-core GEMM.  in_dtype: DT_BF16 or DT_F16; out_dtype: same as the
// input, or DT_F32.  bias may be null; bias_f32 says whether it is fp32.
// aux_mode / act: see the enums at the top of this file.  beta != 0 adds the
// result onto the existing contents of C.  A batch stride of 0 broadcasts.
GB_EXPORT int gb_gemm16(const void* A, const void* B, void* C, const void* bias, int bias_f32,
                        void* aux, int M, int N, int K, int batch, int transA, int transB,
                        long long lda, long long ldb, long long ldc, long long ldaux,
                        long long sA, long long sB, long long sC, long long sAux, int in_dtype,
                        int out_dtype, int act, int aux_mode, int beta, float alpha, int force_bn,
                        void* workspace, long long workspace_bytes, void* stream) {
  if (in_dtype != DT_BF16 && in_dtype != DT_F16) {
    gbh::set_error("gb_gemm16: inputs must be bf16 or fp16");
    return gbh::E_BAD_ARG;
  }
  // contiguous-dimension pitch must be a multiple of 16 bytes for TMA
  if ((lda & 7) || (ldb & 7) || (batch > 1 && ((sA & 7) || (sB & 7)))) {
    gbh::set_error("gb_gemm16: lda/ldb/batch strides must be multiples of 8 elements (got %lld %lld %lld %lld)",
                   lda, ldb, sA, sB);
    return gbh::E_BAD_ARG;
  }
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.C = C; a.bias = bias; a.aux = aux; a.bias_f32 = bias_f32;
  a.ldc = ldc; a.ldaux = ldaux; a.strideC = sC; a.strideAux = sAux;
  a.act = act; a.aux_mode = aux ? aux_mode : AUX_NONE; a.beta = beta; a.alpha = alpha;
  a.out_kind = out_dtype == DT_F32 ? OUT_F32 : (out_dtype == DT_BF16 ? OUT_BF16 : OUT_F16);
  a.in_bf16 = in_dtype == DT_BF16;
  return gemm_tc(2, A, B, a, transA, transB, lda, ldb, sA, sB, force_bn, (cudaStream_t)stream, workspace,
                 workspace_bytes);
}

// int8 x int8 -> int32 GEMM with the dequantising epilogue of the reference's
// quantised Linear (quant/linear.go:110-148):
//   y[m,n] = sx * sw[n] * (acc[m,n] - zx * rowsum[n]) + bias[n]
// A is (M,K) int8 row-major, B is (N,K) int8 row-major.  sx / zx are device
// scalars so that dynamic quantisation needs no host round trip.
GB_EXPORT int gb_gemm_i8(const void* A, const void* B, void* C, const float* bias, int M, int N,
                         int K, long long lda, long long ldb, long long ldc, const float* sx,
                         const int* zx, const float* sw, int per_channel, const int* rowsum,
                         int out_dtype, void* stream) {
  if ((lda & 15) || (ldb & 15)) {
    gbh::set_error("gb_gemm_i8: lda/ldb must be multiples of 16 elements");
    return gbh::E_BAD_ARG;
  }
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = K; a.batch = 1;
  a.C = C; a.bias = bias; a.bias_f32 = 1;
  a.ldc = ldc; a.alpha = 1.f;
  a.out_kind = out_dtype == DT_F32 ? OUT_F32 : (out_dtype == DT_BF16 ? OUT_BF16 : OUT_F16);
  a.in_bf16 = 1;
  a.q_sx = sx; a.q_zx = zx; a.q_sw = sw; a.q_rowsum = rowsum; a.q_per_channel = per_channel;
  return gemm_tc(1, A, B, a, 0, 1, lda, ldb, 0, 0, 0, (cudaStream_t)stream);
}

// fp32 / fp64 SIMT GEMM (exact-precision paths).
GB_EXPORT int gb_gemm_simt(const void* A, const void* B, void* C, int M, int N, int K, int batch,
                           int transA, int transB, long long lda, long long ldb, long long ldc,
                           long long sA, long long sB, long long sC, int dtype, double alpha,
                           int beta, void* stream) {
  dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
  if (grid.y > 65535 || grid.z > 65535) {
    gbh::set_error("gb_gemm_simt: problem too large for this fallback");
    return gbh::E_TOO_LARGE;
  }
  if (dtype != DT_F32 && dtype != DT_F64) {
    gbh::set_error("gb_gemm_simt: dtype must be fp32 or fp64");
    return gbh::E_BAD_ARG;
  }
  if (g_simt_tiled) {
    // the large tile needs enough tiles to occupy the SMs; otherwise 64 x 64 tiles
    const long long big_n = dtype == DT_F32 ? 128 : 64;
    const long long big_tiles = ((M + 127) / 128) * ((N + big_n - 1) / big_n) * (long long)batch;
    const bool big = big_tiles >= 120;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DT_F32) {
      if (big) launch_simt_tiled<float, 8, 8, 16>(A, B, C, M, N, K, batch, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta, st);
      else launch_simt_tiled<float, 4, 4, 16>(A, B, C, M, N, K, batch, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta, st);
    } else {
      if (big) launch_simt_tiled<double, 8, 4, 8>(A, B, C, M, N, K, batch, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta, st);
      else launch_simt_tiled<double, 4, 4, 8>(A, B, C, M, N, K, batch, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta, st);
    }
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  if (dtype == DT_F32) {
    gemm_simt_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const float*)A, (const float*)B, (float*)C, M, N, K, transA, transB, lda, ldb, ldc, sA, sB,
        sC, (float)alpha, beta);
  } else if (dtype == DT_F64) {
    gemm_simt_kernel<double><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const double*)A, (const double*)B, (double*)C, M, N, K, transA, transB, lda, ldb, ldc, sA,
        sB, sC, alpha, beta);
  } else {
    gbh::set_error("gb_gemm_simt: dtype must be fp32 or fp64");
    return gbh::E_BAD_ARG;
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
