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
// Kernel structure (one persistent CTA per SM, 320 threads):
//   warp 0     TMA producer: fills a ring of shared-memory stages
//   warp 1     MMA issuer: one lane issues tcgen05.mma, commits to mbarriers
//   warps 2-9  epilogue: tcgen05.ld the accumulator, apply bias / activation /
//              auxiliary tensor, store to global (two warps per TMEM lane quarter)
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the MMAs
// of tile i+1.
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
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ +
                                    3 * 2 * 256 * 4 /*per-column epilogue constants*/;
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

// ESZ: operand element size (2 = bf16/fp16, 1 = int8).  A_MN / B_MN: operand
// is MN-major.  BN: tile width.
template <int ESZ, bool A_MN, bool B_MN, int BN, int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmArgs args) {
  using C = Cfg<ESZ, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * C::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* s_bias = (float*)((uint8_t*)bars + 256);  // [2][256]
  float* s_qsw = s_bias + 512;                     // [2][256]
  int* s_qrs = (int*)(s_qsw + 512);                // [2][256]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (args.K + C::BK - 1) / C::BK;
  const int tiles_per_batch = args.num_m * args.num_n;
  const int num_tiles = tiles_per_batch * args.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], EW);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
        const int b = t / tiles_per_batch;
        const int r = t - b * tiles_per_batch;
        int mb, nb;
        tile_coords(r, args.num_m, args.num_n, args.group_m, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; kb++) {
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
      for (int kb = 0; kb < num_kb; kb++) {
        ok = mbar_wait(&full_bar[stage], phase, abort_flag, args.status, ST_GEMM_TIMEOUT, 3);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
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
              tc_mma_i8(d_tmem, adesc, bdesc, id, (kb | k) != 0);
            else
              tc_mma_f16(d_tmem, adesc, bdesc, id, (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);
          if (kb == num_kb - 1) tc_commit(&tfull_bar[buf]);
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    // Two warps per TMEM lane quarter; each handles half of the tile's columns.
    // Everything that does not depend on the accumulator (bias, residual / saved
    // pre-activation) is fetched BEFORE waiting for the MMAs, so those latencies
    // overlap the main loop of the tile.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // which column part this warp owns
    const int et = threadIdx.x - 64;  // 0..255 among the epilogue threads
    constexpr int COLS = BN / (EW / 4);  // columns per thread per tile
    constexpr int NCH = COLS / 32;
    uint32_t tphase[2] = {0, 0};
    int local_tile = 0;
    const bool vec_ok = ((args.ldc & 7) == 0) && ((args.strideC & 7) == 0) &&
                        (((uintptr_t)args.C & 15) == 0);
    const bool aux_vec_ok = args.aux_mode == AUX_NONE ||
                            (((args.ldaux & 7) == 0) && ((args.strideAux & 7) == 0) &&
                             (((uintptr_t)args.aux & 15) == 0));
    const bool aux_in = args.aux_mode != AUX_NONE && args.aux_mode != AUX_STORE_PRE;
    const bool has_cols = args.bias != nullptr || ESZ == 1;
    float q_sx = 1.f;
    int q_zx = 0;
    if (ESZ == 1) {
      q_sx = *args.q_sx;
      q_zx = args.q_zx ? *args.q_zx : 0;
    }
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local_tile++) {
      const int buf = local_tile & 1;
      const int b = t / tiles_per_batch;
      const int r = t - b * tiles_per_batch;
      int mb, nb;
      tile_coords(r, args.num_m, args.num_n, args.group_m, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
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
      ok = mbar_wait(&tfull_bar[buf], tphase[buf], abort_flag, args.status, ST_GEMM_TIMEOUT, 4);
      if (!ok) break;
      tphase[buf] ^= 1;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * COLS;
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
      // accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
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

int g_epi_warps = 8;

template <int ESZ, bool A_MN, bool B_MN, int BN, int EW>
int launch_tc_ew(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
                 cudaStream_t stream) {
  using C = Cfg<ESZ, BN>;
  auto kern = gemm_tcgen05_kernel<ESZ, A_MN, B_MN, BN, EW>;
  static bool configured = false;
  if (!configured) {
    GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  int tiles = args.num_m * args.num_n * args.batch;
  int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, 64 + 32 * EW, C::SMEM_BYTES, stream>>>(tmA, tmB, args);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <int ESZ, bool A_MN, bool B_MN, int BN>
int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
              cudaStream_t stream) {
  if (g_epi_warps == 4) return launch_tc_ew<ESZ, A_MN, B_MN, BN, 4>(tmA, tmB, args, num_sms, stream);
  return launch_tc_ew<ESZ, A_MN, B_MN, BN, 8>(tmA, tmB, args, num_sms, stream);
}

template <int ESZ, int BN>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                   const GemmArgs& args, int num_sms, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_tc<ESZ, false, false, BN>(tmA, tmB, args, num_sms, stream);
  if (ESZ == 2) {
    if (!a_mn && b_mn) return launch_tc<2, false, true, BN>(tmA, tmB, args, num_sms, stream);
    if (a_mn && !b_mn) return launch_tc<2, true, false, BN>(tmA, tmB, args, num_sms, stream);
    return launch_tc<2, true, true, BN>(tmA, tmB, args, num_sms, stream);
  }
  gbh::set_error("int8 GEMM supports only A (M,K) row-major with B (N,K) row-major");
  return gbh::E_BAD_ARG;
}

int g_num_sms = 0;
int g_group_m = 8;

// Builds the two tensor maps and launches.  esz: 2 (bf16/fp16) or 1 (int8).
int gemm_tc(int esz, const void* A, const void* B, GemmArgs& args, int transA, int transB,
            long long lda, long long ldb, long long sA, long long sB, int force_bn,
            cudaStream_t stream) {
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
  args.num_m = (M + BM - 1) / BM;
  args.num_n = (N + bn - 1) / bn;
  args.status = gbh::status_ptr();
  args.group_m = g_group_m;

  CUtensorMapDataType dt = esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : (args.in_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUtensorMap tmA, tmB;
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
  if (esz == 2) {
    if (bn == 256) return dispatch_major<2, 256>(a_mn, b_mn, tmA, tmB, args, g_num_sms, stream);
    return dispatch_major<2, 128>(a_mn, b_mn, tmA, tmB, args, g_num_sms, stream);
  }
  if (bn == 256) return dispatch_major<1, 256>(a_mn, b_mn, tmA, tmB, args, g_num_sms, stream);
  return dispatch_major<1, 128>(a_mn, b_mn, tmA, tmB, args, g_num_sms, stream);
}

}  // namespace

// Tuning knobs: epilogue warps (4 or 8) and rasterisation group height (row blocks).
GB_EXPORT int gb_gemm_tune(int epi_warps, int group_m) {
  if (epi_warps == 4 || epi_warps == 8) g_epi_warps = epi_warps;
  if (group_m >= 1) g_group_m = group_m;
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
                        void* stream) {
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
  return gemm_tc(2, A, B, a, transA, transB, lda, ldb, sA, sB, force_bn, (cudaStream_t)stream);
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
