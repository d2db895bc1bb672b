// Flash attention for sm_100a: forward and backward on tcgen05 tensor cores
// with the score tile, the probability tile and the output accumulator in
// tensor memory.
//
// Math follows the reference's fused kernels (backend/cuda/gonn_cuda.cu:302-450
// forward with online softmax and L = m + log(l); :333-383 backward identities
// p = exp(s*scale - L), D = dO.O, dV += p^T dO, dS = p (dO.v - D) scale,
// dQ += dS k, dK += dS^T q) and the scale 1/sqrt(d) and causal rule k <= q of
// nn/attention.go:124-147.  The design is new: 128-row tiles, bf16/fp16 operands,
// fp32 accumulation, no atomics (dQ and dK/dV are produced by two kernels so that
// every output tile has one owner and a fixed summation order).
//
// Forward CTA (192 threads, two CTAs per SM) owns 128 query rows of one (batch, head):
//   warp 0      TMA loads of Q once and the K / V sub-tiles of 64 keys (rings)
//   warp 1      MMA issue: S = Q K^T into one of two TMEM score buffers, then
//               O += P V with P read from TMEM (written there by the softmax warps)
//   warps 2-5   softmax: one thread per row; running max / sum in registers;
//               O is rescaled only when the max moved by more than 2^8
// Backward: a row-statistics kernel (Delta = dO . O), then one CTA per 128-key tile for
// dK / dV and one CTA per 128-query tile for dQ; both stream 64-row sub-tiles, keep S and dP
// in TMEM (two buffers and sixteen elementwise warps at head_dim 128; one buffer, eight
// warps and two CTAs per SM at head_dim 64) and feed P^T / dS^T back to the tensor core as
// TMEM A operands.
// Tensors are addressed through 4-D tensor maps (d, s, h, b) with arbitrary
// strides, so (B,S,H,D) and (B,H,S,D) layouts both work without copies.
#include "common.cuh"

#include <type_traits>

using namespace gb;

namespace {

constexpr int BQ = 128;   // query rows per tile
constexpr int BKV = 128;  // key rows per tile
constexpr int kFwdThreads = 192;

struct AttnArgs {
  int B, H, Sq, Sk;
  int D;  // the tensors' head size: a multiple of 8, at most the kernel's HD (TMA zero-fills the rest)
  float scale_log2;  // scale * log2(e)
  float scale;
  int causal;
  int in_bf16;
  // element strides of O / dO / dQ / dK / dV style tensors: (b, s, h); d is contiguous
  long long o_sb, o_ss, o_sh;
  void* O;
  float* LSE;  // [B, H, Sq]
  // backward
  const float* Delta;  // [B, H, Sq]
  void* dQ; void* dK; void* dV;
  long long dq_sb, dq_ss, dq_sh;
  long long dk_sb, dk_ss, dk_sh;
  long long dv_sb, dv_ss, dv_sh;
  // optional spill of dS^T from the dK/dV kernel: [B*H][ds_rows keys][ds_ld queries], 16-bit, already
  // multiplied by the softmax scale.  When set, dQ is one product of this matrix with K
  // (fa_bwd_dq_ds_kernel) instead of a second pass that recomputes S, P and dP.
  void* dS;
  long long ds_ld, ds_rows;
  int* status;
  // optional timeline of CTA (0,0,0) of the dK/dV kernel: [3 lanes][kTraceSlots] SM clock stamps
  long long* trace;
};

constexpr int kTraceSlots = 512;
// lane: 0 = MMA thread, 1 / 2 = first warp of elementwise group 0 / 1
// Compiled in only with -DGB_FA_TRACE: the pointer and the counter cost three registers in a kernel
// that sits at its register cap.
__device__ __forceinline__ void trace_stamp(long long* trace, int lane_id, int& n) {
#ifdef GB_FA_TRACE
  if (trace && n < kTraceSlots) trace[lane_id * kTraceSlots + n++] = clock64();
#else
  (void)trace; (void)lane_id; (void)n;
#endif
}

// One 32-byte store (a whole DRAM sector) from eight registers; the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t a4, uint32_t a5, uint32_t a6, uint32_t a7) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a0), "r"(a1), "r"(a2),
               "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7)
               : "memory");
}

__device__ __forceinline__ uint32_t pack16(float a, float b, int bf) {
  return bf ? pack_bf16(a, b) : pack_f16(a, b);
}

// Stores `n` fp32 values (n multiple of 8) as 16-bit to a 16-byte aligned row.
template <int N>
__device__ __forceinline__ void store_row16(void* dst, const float* v, int bf) {
#pragma unroll
  for (int j = 0; j < N; j += 8) {
    uint4 o;
    o.x = pack16(v[j], v[j + 1], bf);
    o.y = pack16(v[j + 2], v[j + 3], bf);
    o.z = pack16(v[j + 4], v[j + 5], bf);
    o.w = pack16(v[j + 6], v[j + 7], bf);
    *reinterpret_cast<uint4*>((uint16_t*)dst + j) = o;
  }
}

// The same for a row of which only `ncols` columns (a multiple of 8, counted from this pointer)
// exist in memory: head sizes below the kernel's compile-time HD.
template <int N>
__device__ __forceinline__ void store_row16_lim(void* dst, const float* v, int bf, int ncols) {
  if (ncols >= N) {
    store_row16<N>(dst, v, bf);
    return;
  }
#pragma unroll
  for (int j = 0; j < N; j += 8) {
    if (j < ncols) {
      uint4 o;
      o.x = pack16(v[j], v[j + 1], bf);
      o.y = pack16(v[j + 2], v[j + 3], bf);
      o.z = pack16(v[j + 4], v[j + 5], bf);
      o.w = pack16(v[j + 6], v[j + 7], bf);
      *reinterpret_cast<uint4*>((uint16_t*)dst + j) = o;
    }
  }
}

constexpr int BKF = 64;  // key rows per forward sub-tile

// Forward tiling: 128 query rows per CTA, keys in 64-row sub-tiles.  Two score buffers of 64
// columns and the output accumulator need 128 + HD <= 256 TMEM columns, and the shared
// memory of one CTA stays under half an SM, so two CTAs share an SM: while the softmax warps
// of one are busy, the tensor core serves the other.
template <int HD>
struct FwdCfg {
  static constexpr int CH = HD / 64;                   // 64-column chunks per row
  static constexpr int Q_BYTES = CH * BQ * 128;        // the resident query tile
  static constexpr int SUB_BYTES = CH * BKF * 128;     // one K or V sub-tile
  static constexpr int STAGES = HD == 64 ? 3 : 2;
  static constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * SUB_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 256;
  static constexpr int COL_S0 = 0, COL_S1 = 64, COL_O = 128;
};

template <int HD, bool BF>
__global__ void __launch_bounds__(kFwdThreads, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const AttnArgs args) {
  using C = FwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;                   // [STAGES]
  uint8_t* sV = sK + C::STAGES * C::SUB_BYTES;     // [STAGES]
  uint64_t* bars = (uint64_t*)(sV + C::STAGES * C::SUB_BYTES);
  uint64_t* q_full = bars;                    // 1
  uint64_t* k_full = bars + 1;                // STAGES
  uint64_t* k_empty = k_full + C::STAGES;     // STAGES
  uint64_t* v_full = k_empty + C::STAGES;     // STAGES
  uint64_t* v_empty = v_full + C::STAGES;     // STAGES
  uint64_t* s_full = v_empty + C::STAGES;     // 2
  uint64_t* p_full = s_full + 2;              // 2
  uint64_t* pv_done = p_full + 2;             // 2
  uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (args.Sq + BQ - 1) / BQ;
  // heavy (late) query tiles first when causal
  const int q_tile = args.causal ? (num_q_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * BQ;
  int n_kv = (args.Sk + BKF - 1) / BKF;
  if (args.causal) n_kv = min(n_kv, (q_tile + 1) * (BQ / BKF));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::STAGES; i++) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp
      mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    if (elect_one()) {
      mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::CH; c++) tma_load_4d(sQ + c * BQ * 128, &tmQ, q_full, c * 64, q0, h, b);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_kv; j++) {
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 1)) break;
        mbar_expect_tx(&k_full[st], C::SUB_BYTES);
#pragma unroll
        for (int c = 0; c < C::CH; c++)
          tma_load_4d(sK + st * C::SUB_BYTES + c * BKF * 128, &tmK, &k_full[st], c * 64, j * BKF, h, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 2)) break;
        mbar_expect_tx(&v_full[st], C::SUB_BYTES);
#pragma unroll
        for (int c = 0; c < C::CH; c++)
          tma_load_4d(sV + st * C::SUB_BYTES + c * BKF * 128, &tmV, &v_full[st], c * 64, j * BKF, h, b);
        if (++st == C::STAGES) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t fmt = BF ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(1u, fmt, false, false, BQ, BKF);
      const uint32_t idesc_o = make_idesc(1u, fmt, false, true, BQ, HD);
      const uint32_t qa = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 3);
      int st_s = 0;
      uint32_t ph_s = 0;
      auto issue_s = [&](int j) {
        if (!mbar_wait(&k_full[st_s], ph_s, abort_flag, args.status, ST_ATTN_TIMEOUT, 4)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(sK + st_s * C::SUB_BYTES);
        const uint32_t d = tmem_base + ((j & 1) ? C::COL_S1 : C::COL_S0);
#pragma unroll
        for (int k = 0; k < HD / 16; k++)
          tc_mma_f16(d, make_smem_desc_sw128(qa + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024),
                     make_smem_desc_sw128(ka + (k / 4) * (BKF * 128) + (k % 4) * 32, 16, 1024), idesc_s, k != 0);
        tc_commit(&k_empty[st_s]);
        tc_commit(&s_full[j & 1]);
        if (++st_s == C::STAGES) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      if (ok && n_kv > 0) ok = issue_s(0);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_kv && ok; j++) {
        if (j + 1 < n_kv) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int sb = j & 1;
        ok = mbar_wait(&p_full[sb], (j >> 1) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 5);
        if (!ok) break;
        ok = mbar_wait(&v_full[st], ph, abort_flag, args.status, ST_ATTN_TIMEOUT, 6);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(sV + st * C::SUB_BYTES);
        const uint32_t p_tmem = tmem_base + (sb ? C::COL_S1 : C::COL_S0);
        const uint32_t d = tmem_base + C::COL_O;
#pragma unroll
        for (int k = 0; k < BKF / 16; k++) {
          // V is the MN-major B operand: 64-wide d chunks are BKF*128 B apart, 8-row groups
          // 1024 B apart, one MMA step covers 16 key rows.
          tc_mma_f16_ts(d, p_tmem + k * 8, make_smem_desc_sw128(va + k * 16 * 128, BKF * 128, 1024), idesc_o,
                        (j | k) != 0);
        }
        tc_commit(&v_empty[st]);
        tc_commit(&pv_done[sb]);
        if (++st == C::STAGES) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax warps ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row inside the tile
    const int qrow = q0 + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m_used = -INFINITY;  // in log2 units, already scaled
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; j++) {
      const int sb = j & 1;
      ok = mbar_wait(&s_full[sb], (j >> 1) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 7);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + (sb ? C::COL_S1 : C::COL_S0);
      const int kv0 = j * BKF;
      // this warp's 32 rows start at q0 + 32 * quarter: a sub-tile entirely to the right of
      // them contributes nothing (P = 0, running max and sum unchanged)
      if (args.causal && kv0 > q0 + quarter * 32 + 31) {
        uint32_t zero[32];
#pragma unroll
        for (int i = 0; i < 32; i++) zero[i] = 0u;
        tmem_st32(s_addr, zero);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[sb]);
        continue;
      }
      uint32_t rr[BKF];
      tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&rr[0]));
      tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&rr[32]));
      tmem_ld_wait();
      float s[BKF];
#pragma unroll
      for (int i = 0; i < BKF; i++) s[i] = __uint_as_float(rr[i]);
      const bool need_mask = (args.causal && kv0 + BKF - 1 > q0 + quarter * 32) || (kv0 + BKF > args.Sk);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BKF; c++) {
          const int kv = kv0 + c;
          if (kv >= args.Sk || (args.causal && kv > qrow)) s[c] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < BKF; c++) mx = fmaxf(mx, s[c]);
      float m_new = fmaxf(m_used, mx * args.scale_log2);
      if (m_new == -INFINITY) m_new = 0.f;
      // rescale O only when the running max moved by more than 8 (a factor 256)
      const bool need = (m_new - m_used) > 8.f;
      float alpha = 1.f;
      if (need) {
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 8);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; c++) {
          uint32_t ro[32];
          tmem_ld32(lane_addr + C::COL_O + c * 32, ro);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
          tmem_st32(lane_addr + C::COL_O + c * 32, ro);
        }
        tmem_st_wait();
      }
      float sum = 0.f;
      uint32_t pk[BKF / 2];
#pragma unroll
      for (int i = 0; i < BKF / 2; i++) {
        const float p0 = exp2f(fmaf(s[2 * i], args.scale_log2, -m_used));
        const float p1 = exp2f(fmaf(s[2 * i + 1], args.scale_log2, -m_used));
        sum += p0 + p1;
        pk[i] = BF ? pack_bf16(p0, p1) : pack_f16(p0, p1);
      }
      tmem_st32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
    }
    if (ok && n_kv > 0)
      ok = mbar_wait(&pv_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 9);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < args.Sq;
      uint16_t* orow = (uint16_t*)args.O + (long long)b * args.o_sb + (long long)qrow * args.o_ss +
                       (long long)h * args.o_sh;
#pragma unroll
      for (int c = 0; c < HD / 32; c++) {
        uint32_t ro[32];
        if (n_kv > 0) {
          tmem_ld32(lane_addr + C::COL_O + c * 32, ro);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) ro[i] = 0;
        }
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(ro[i]) * inv;
        if (row_ok) store_row16_lim<32>(orow + c * 32, v, BF, args.D - c * 32);
      }
      if (row_ok && args.LSE) {
        // natural-log LSE of the scaled scores
        args.LSE[((long long)b * args.H + h) * args.Sq + qrow] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d]  (fp32), one warp per row
template <typename T>
__global__ void fa_delta_kernel(const T* __restrict__ O, const T* __restrict__ dO,
                                float* __restrict__ delta, int B, int H, int S, int D,
                                long long o_sb, long long o_ss, long long o_sh, long long g_sb,
                                long long g_ss, long long g_sh) {
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)B * H * S;
  for (long long i = (long long)blockIdx.x * warps + warp; i < total; i += (long long)gridDim.x * warps) {
    const int q = (int)(i % S);
    const int h = (int)((i / S) % H);
    const int b = (int)(i / ((long long)S * H));
    const T* o = O + b * o_sb + q * o_ss + h * o_sh;
    const T* g = dO + b * g_sb + q * g_ss + h * g_sh;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += (float)o[d] * (float)g[d];
    s = warp_sum(s);
    if (lane == 0) delta[i] = s;
  }
}


// The same for 16-byte aligned rows of D = 8 * TPR elements: TPR threads per row, one
// 16-byte load of O and of dO each.
template <typename T, int TPR>
__global__ void __launch_bounds__(256)
fa_delta_vec_kernel(const T* __restrict__ O, const T* __restrict__ dO, float* __restrict__ delta, int B,
                    int H, int S, long long o_sb, long long o_ss, long long o_sh, long long g_sb,
                    long long g_ss, long long g_sh) {
  const long long total = (long long)B * H * S;
  const int sub = threadIdx.x % TPR;
  constexpr int RPB = 256 / TPR;  // rows per CTA pass; every thread of the CTA runs the same trip count
  for (long long base = (long long)blockIdx.x * RPB; base < total; base += (long long)gridDim.x * RPB) {
    const long long i = base + threadIdx.x / TPR;
    // rows are visited in (b, s, h) order so that neighbouring threads read neighbouring memory
    const bool live = i < total;
    const long long ii = live ? i : 0;
    const int h = (int)(ii % H);
    const int q = (int)((ii / H) % S);
    const int b = (int)(ii / ((long long)S * H));
    const uint4 uo = *reinterpret_cast<const uint4*>(O + b * o_sb + q * o_ss + h * o_sh + sub * 8);
    const uint4 ug = *reinterpret_cast<const uint4*>(dO + b * g_sb + q * g_ss + h * g_sh + sub * 8);
    const T* eo = reinterpret_cast<const T*>(&uo);
    const T* eg = reinterpret_cast<const T*>(&ug);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) s += (float)eo[j] * (float)eg[j];
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (live && sub == 0) delta[((long long)b * H + h) * S + q] = s;
  }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
constexpr int kBwdThreadsMax = 64 + 16 * 32;     // TMA warp, MMA warp, up to sixteen elementwise warps
constexpr int BSUB = 64;                  // rows of one streamed sub-tile

// Backward tiling.  The resident operand pair is a 128-row tile; the streamed pair comes in
// 64-row sub-tiles through a ring of NS stages.  Scores and dP of a sub-tile are 128 x 64
// fp32 blocks in TMEM, double buffered, so the tensor core computes sub-tile i+1 (and the
// accumulations of sub-tile i-1) while the elementwise warps work on sub-tile i.  The
// elementwise warps form two groups of eight; group g owns TMEM buffer g and every second
// sub-tile, so the TMEM round trips of one group hide behind the arithmetic of the other.
template <int HD, bool DUAL_>
struct BwdCfg {
  static constexpr int CH = HD / 64;
  static constexpr int TILE_BYTES = CH * 128 * 128;
  static constexpr int SUB_BYTES = CH * BSUB * 128;
  static constexpr int NS = 4;
  static constexpr int STAT_BYTES = NS * 2 * BSUB * 4;  // per stage: 64 x LSE*log2(e), 64 x Delta*scale
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + NS * 2 * SUB_BYTES + STAT_BYTES + 1024 + 256;
  // head_dim 64: one S/dP buffer, eight elementwise warps, 256 TMEM columns and < 113 KB of
  // shared memory, so TWO CTAs share an SM and hide each other's serial chain (S/dP MMAs ->
  // elementwise -> accumulation MMAs) as well as each other's start-up and epilogue.
  // head_dim 128: the accumulators alone need 256 columns, so one CTA per SM with two S/dP
  // buffers and two groups of eight elementwise warps that own alternate sub-tiles.
  static constexpr bool DUAL = DUAL_;
  static_assert(!DUAL_ || HD == 64, "two CTAs per SM need head_dim 64");
  static constexpr int NBUF = DUAL ? 1 : 2;
  static constexpr int EW = 8 * NBUF;
  static constexpr int THREADS = 64 + EW * 32;
  static constexpr int CTAS_PER_SM = DUAL ? 2 : 1;
  static constexpr int TMEM_COLS = DUAL ? 256 : 512;
  // buffer b: scores at b*128, dP at b*128 + 64; accumulators behind them
  static constexpr int COL_ACC0 = 128 * NBUF, COL_ACC1 = COL_ACC0 + HD;
  // resident A operands kept in TMEM where the columns allow it
  static constexpr bool KV_IN_TMEM = HD == 64 && !DUAL;
  static constexpr bool Q_IN_TMEM = !DUAL;
  static constexpr int COL_KT = COL_ACC0 + 2 * HD, COL_VT = COL_KT + HD / 2;
  static constexpr int COL_QT = COL_ACC0 + HD, COL_GT = COL_QT + HD / 2;
};

// K-major operand descriptor for step k (16 columns) of a [128 x HD] tile
__device__ __forceinline__ uint64_t kdesc(uint32_t base, int k) {
  return make_smem_desc_sw128(base + (k / 4) * (128 * 128) + (k % 4) * 32, 16, 1024);
}
// the same for a [64 x HD] sub-tile (64-column chunks are 64 rows apart)
__device__ __forceinline__ uint64_t kdesc_sub(uint32_t base, int k) {
  return make_smem_desc_sw128(base + (k / 4) * (BSUB * 128) + (k % 4) * 32, 16, 1024);
}
// MN-major operand descriptor for step k (16 rows) of a [64 rows x HD] sub-tile
__device__ __forceinline__ uint64_t mndesc_sub(uint32_t base, int k) {
  return make_smem_desc_sw128(base + k * 16 * 128, BSUB * 128, 1024);
}

// Copies this thread's row of a resident [128 x HD] 16-bit tile (128-byte swizzled rows in
// 64-column chunks of 128 rows) into TMEM columns [col, col + HD / 2): the layout of an A
// operand read from tensor memory, so the MMAs that use the tile stop re-reading it from
// shared memory on every step.
template <int HD>
__device__ __forceinline__ void tile_row_to_tmem(const uint8_t* tile, int r, uint32_t lane_addr, uint32_t col) {
#pragma unroll
  for (int c = 0; c < HD / 64; c++) {
    uint32_t w[32];
    const uint32_t row = smem_u32(tile + c * 128 * 128 + r * 128);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      uint4 u;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                   : "r"(row + (((uint32_t)j ^ ((uint32_t)r & 7u)) << 4)));
      w[4 * j] = u.x; w[4 * j + 1] = u.y; w[4 * j + 2] = u.z; w[4 * j + 3] = u.w;
    }
    tmem_st32(lane_addr + col + c * 32, w);
  }
  tmem_st_wait();
}

template <bool BF>
__device__ __forceinline__ uint32_t pack16t(float a, float b) {
  return BF ? pack_bf16(a, b) : pack_f16(a, b);
}

// dK / dV: one CTA per 128-key tile; streams 64-row query sub-tiles.  Works in the
// transposed domain (rows = keys) so that P^T and dS^T are A operands in TMEM.
template <int HD, bool BF, bool DUAL>
__global__ void __launch_bounds__(BwdCfg<HD, DUAL>::THREADS, BwdCfg<HD, DUAL>::CTAS_PER_SM)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                  const AttnArgs args) {
  using C = BwdCfg<HD, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::TILE_BYTES;
  uint8_t* ring = sV + C::TILE_BYTES;  // [NS] x {Q sub-tile, dO sub-tile}
  float* sStat = (float*)(ring + C::NS * 2 * C::SUB_BYTES);  // [NS][2][64]
  uint64_t* bars = (uint64_t*)((uint8_t*)sStat + C::STAT_BYTES);
  uint64_t* kv_full = bars;                 // 1
  uint64_t* q_full = bars + 1;              // NS
  uint64_t* q_empty = q_full + C::NS;       // NS
  uint64_t* sdp_full = q_empty + C::NS;     // 2
  uint64_t* p_full = sdp_full + 2;          // 2
  uint64_t* acc_done = p_full + 2;          // 1
  uint64_t* a_ready = acc_done + 1;         // 1: K and V copied into TMEM
  uint32_t* tmem_slot = (uint32_t*)(a_ready + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kv0 = kv_tile * BKV;
  const int num_sub = (args.Sq + BSUB - 1) / BSUB;
  const int i_begin = args.causal ? kv_tile * (BKV / BSUB) : 0;
  const int n_it = max(num_sub - i_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < C::NS; i++) {
      mbar_init(&q_full[i], 1 + 32);  // the TMA transaction + the 32 lanes that stage the row statistics
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < 2; i++) { mbar_init(&sdp_full[i], 1); mbar_init(&p_full[i], 8); }
    mbar_init(acc_done, 1);
    mbar_init(a_ready, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: TMA for the tiles (lane 0), row statistics by all lanes ----
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::CH; c++) {
        tma_load_4d(sK + c * 128 * 128, &tmK, kv_full, c * 64, kv0, h, b);
        tma_load_4d(sV + c * 128 * 128, &tmV, kv_full, c * 64, kv0, h, b);
      }
    }
    const float* stat_g = (lane < 16 ? args.LSE : args.Delta) + ((long long)b * args.H + h) * args.Sq;
    const bool vec = (args.Sq & 3) == 0;
    int st = 0;
    uint32_t ph = 0;
    for (int it = 0; it < n_it; it++) {
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&q_empty[st], ph ^ 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 11);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int q0 = (i_begin + it) * BSUB;
      if (lane == 0) {
        mbar_expect_tx(&q_full[st], 2 * C::SUB_BYTES);
        uint8_t* sQ = ring + st * 2 * C::SUB_BYTES;
        uint8_t* sdO = sQ + C::SUB_BYTES;
#pragma unroll
        for (int c = 0; c < C::CH; c++) {
          tma_load_4d(sQ + c * BSUB * 128, &tmQ, &q_full[st], c * 64, q0, h, b);
          tma_load_4d(sdO + c * BSUB * 128, &tmdO, &q_full[st], c * 64, q0, h, b);
        }
      }
      // lanes 0-15: LSE * log2(e) (rows past the end and fully masked rows read +inf, so
      // their probabilities come out 0); lanes 16-31: Delta * scale
      const int qs = q0 + (lane & 15) * 4;
      float4 t;
      if (vec && qs + 4 <= args.Sq) {
        t = __ldg(reinterpret_cast<const float4*>(stat_g + qs));
      } else {
        const float fill = lane < 16 ? INFINITY : 0.f;
        t.x = qs < args.Sq ? __ldg(stat_g + qs) : fill;
        t.y = qs + 1 < args.Sq ? __ldg(stat_g + qs + 1) : fill;
        t.z = qs + 2 < args.Sq ? __ldg(stat_g + qs + 2) : fill;
        t.w = qs + 3 < args.Sq ? __ldg(stat_g + qs + 3) : fill;
      }
      if (lane < 16) {
        const float k = 1.4426950408889634f;
        t.x = t.x == -INFINITY ? INFINITY : t.x * k;
        t.y = t.y == -INFINITY ? INFINITY : t.y * k;
        t.z = t.z == -INFINITY ? INFINITY : t.z * k;
        t.w = t.w == -INFINITY ? INFINITY : t.w * k;
      } else {
        t.x *= args.scale; t.y *= args.scale; t.z *= args.scale; t.w *= args.scale;
      }
      *reinterpret_cast<float4*>(sStat + st * 128 + lane * 4) = t;
      mbar_arrive(&q_full[st]);
      if (++st == C::NS) { st = 0; ph ^= 1; }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t fmt = BF ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(1u, fmt, false, false, 128, BSUB);
      const uint32_t idesc_acc = make_idesc(1u, fmt, false, true, 128, HD);
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      bool ok = mbar_wait(kv_full, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 12);
      if (ok && C::KV_IN_TMEM) {
        ok = mbar_wait(a_ready, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 18);
        tc_fence_after();
      }
      int st_s = 0;        // ring stage of the next S / dP issue
      uint32_t ph_s = 0;
      auto issue_sdp = [&](int it) {
        if (!mbar_wait(&q_full[st_s], ph_s, abort_flag, args.status, ST_ATTN_TIMEOUT, 13)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(ring + st_s * 2 * C::SUB_BYTES), ga = qa + C::SUB_BYTES;
        const uint32_t d = tmem_base + (it % C::NBUF) * 128;
        // two independent accumulation chains, interleaved so that an MMA never has to wait
        // for the one just before it
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          if (C::KV_IN_TMEM) {
            tc_mma_f16_ts(d, tmem_base + C::COL_KT + k * 8, kdesc_sub(qa, k), idesc_s, k != 0);
            tc_mma_f16_ts(d + 64, tmem_base + C::COL_VT + k * 8, kdesc_sub(ga, k), idesc_s, k != 0);
          } else {
            tc_mma_f16(d, kdesc(ka, k), kdesc_sub(qa, k), idesc_s, k != 0);       // S^T = K Q^T
            tc_mma_f16(d + 64, kdesc(va, k), kdesc_sub(ga, k), idesc_s, k != 0);  // dP^T = V dO^T
          }
        }
        tc_commit(&sdp_full[it % C::NBUF]);
        if (++st_s == C::NS) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      long long* tr = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 ? args.trace : nullptr;
      int ntr = 0;
      trace_stamp(tr, 0, ntr);
      if (ok && n_it > 0) ok = issue_sdp(0);
      int st = 0;
      for (int it = 0; it < n_it && ok; it++) {
        // two buffers: the next sub-tile's S / dP are issued before this one's P / dS are
        // awaited; one buffer: they follow this sub-tile's accumulation MMAs
        if (C::NBUF == 2 && it + 1 < n_it) {
          ok = issue_sdp(it + 1);
          if (!ok) break;
        }
        trace_stamp(tr, 0, ntr);  // S / dP of the next sub-tile issued
        const int bb = it % C::NBUF;
        ok = mbar_wait(&p_full[bb], (it / C::NBUF) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 14);
        if (!ok) break;
        trace_stamp(tr, 0, ntr);  // P / dS of this sub-tile ready
        tc_fence_after();
        const uint32_t qa = smem_u32(ring + st * 2 * C::SUB_BYTES), ga = qa + C::SUB_BYTES;
        const uint32_t pt = tmem_base + bb * 128;
        // each elementwise warp left 16 packed columns at the start of its own 32-column
        // range, so MMA step k reads from (k / 2) * 32 + (k % 2) * 8
#pragma unroll
        for (int k = 0; k < BSUB / 16; k++) {
          tc_mma_f16_ts(tmem_base + C::COL_ACC0, pt + (k >> 1) * 32 + (k & 1) * 8, mndesc_sub(ga, k), idesc_acc,
                        (it | k) != 0);  // dV += P^T dO
          tc_mma_f16_ts(tmem_base + C::COL_ACC1, pt + 64 + (k >> 1) * 32 + (k & 1) * 8, mndesc_sub(qa, k),
                        idesc_acc, (it | k) != 0);  // dK += dS^T Q
        }
        tc_commit(&q_empty[st]);
        if (it == n_it - 1) tc_commit(acc_done);
        if (++st == C::NS) st = 0;
        if (C::NBUF == 1 && it + 1 < n_it) ok = issue_sdp(it + 1);
      }
    }
    __syncwarp();
  } else {
    const int e = warp - 2;
    const int group = e >> 3;                // sub-tiles it with it % NBUF == group, TMEM buffer `group`
    const int half = (e >> 2) & 1;           // which 32 of the sub-tile's 64 query columns
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // key row inside the tile
    const int kvrow = kv0 + r;
    const bool row_dead = kvrow >= args.Sk;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t my = lane_addr + group * 128 + half * 32;
    bool ok = true;
    if (C::KV_IN_TMEM && group == 0) {
      // the eight warps of group 0 copy K (half 0) and V (half 1) into TMEM once
      ok = mbar_wait(kv_full, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 19);
      if (ok) {
        tile_row_to_tmem<HD>(half == 0 ? sK : sV, r, lane_addr, half == 0 ? C::COL_KT : C::COL_VT);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
      }
    }
    long long* tr = ((blockIdx.x | blockIdx.y | blockIdx.z) == 0 && (e & 7) == 0 && lane == 0) ? args.trace : nullptr;
    int ntr = 0;
    // where this thread's key row starts in the dS^T spill (its half of each 64-query sub-tile)
    // (a byte offset from args.dS; the workspace is at most 4 GiB, so 32 bits hold it)
    const uint32_t ds_off = (uint32_t)(((((long long)b * args.H + h) * args.ds_rows + kvrow) * args.ds_ld + half * 32) * 2);
    for (int it = group; it < n_it; it += C::NBUF) {
      const int st = it % C::NS;
      trace_stamp(tr, 1 + group, ntr);  // starts waiting
      ok = mbar_wait(&q_full[st], (it / C::NS) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 17);
      if (!ok) break;
      ok = mbar_wait(&sdp_full[group], (it / C::NBUF) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 15);
      if (!ok) break;
      trace_stamp(tr, 1 + group, ntr);  // scores ready
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld32(my, rs);
      tmem_ld32(my + 64, rd);
      const float4* l4 = reinterpret_cast<const float4*>(sStat + st * 128 + half * 32);
      const float4* d4 = reinterpret_cast<const float4*>(sStat + st * 128 + 64 + half * 32);
      tmem_ld_wait();
      trace_stamp(tr, 1 + group, ntr);  // loaded
      const int q0 = (i_begin + it) * BSUB + half * 32;  // first query column of this thread
      // masking is needed on the diagonal sub-tiles and for key rows past the end; the common
      // case runs a loop without any of the compare / select instructions
      // The warp's 32 key rows against its 32 query columns: entirely above the diagonal
      // (everything masked: zeros, no arithmetic), entirely on or below it (no masking), or
      // the 32 x 32 block the diagonal crosses (per-element test).
      const int rel = kv0 + quarter * 32 - q0;  // first key row minus first query column
      const bool all_masked = args.causal && rel > 31;
      const bool masked = __any_sync(0xffffffffu, row_dead) || (args.causal && rel + 31 > 0);
      if (all_masked) {
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; i++) z[i] = 0u;
        tmem_st16(my, z);
        tmem_st16(my + 64, z);
        if (args.dS) {
          uint8_t* dst = (uint8_t*)args.dS + ds_off + (uint32_t)(i_begin + it) * (BSUB * 2);
          st_global_v8(dst, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u);
          st_global_v8(dst + 32, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[group]);
        continue;
      }
      uint32_t pp[16], pd[16];
      auto body = [&](auto use_mask) {
#pragma unroll
        for (int g = 0; g < 8; g++) {
          const float4 l = l4[g], d = d4[g];
          const float ls[4] = {l.x, l.y, l.z, l.w};
          const float ds[4] = {d.x, d.y, d.z, d.w};
          float p[4], q[4];
#pragma unroll
          for (int u = 0; u < 4; u++) {
            const int j = 4 * g + u;
            // head_dim 64: every fourth exponential runs on the FMA pipe, because there the MUFU
            // unit is the busiest resource of this loop (at 128 the tensor core is)
            const float e = fmaf(__uint_as_float(rs[j]), args.scale_log2, -ls[u]);
            p[u] = (HD == 64 && u == 3 && !decltype(use_mask)::value) ? exp2_poly(e) : exp2f(e);
            if (decltype(use_mask)::value) {
              if (row_dead || (args.causal && kvrow > q0 + j)) p[u] = 0.f;
            }
            q[u] = p[u] * fmaf(__uint_as_float(rd[j]), args.scale, -ds[u]);
          }
          pp[2 * g] = pack16t<BF>(p[0], p[1]);
          pp[2 * g + 1] = pack16t<BF>(p[2], p[3]);
          pd[2 * g] = pack16t<BF>(q[0], q[1]);
          pd[2 * g + 1] = pack16t<BF>(q[2], q[3]);
        }
      };
      if (masked) body(std::true_type{});
      else body(std::false_type{});
      // each warp overwrites only columns it has read itself
      trace_stamp(tr, 1 + group, ntr);  // computed
      tmem_st16(my, pp);
      tmem_st16(my + 64, pd);
      if (args.dS) {
        // this thread's key row, its 32 query columns: 64 contiguous bytes of dS^T
        uint8_t* dst = (uint8_t*)args.dS + ds_off + (uint32_t)(i_begin + it) * (BSUB * 2);
        st_global_v8(dst, pd[0], pd[1], pd[2], pd[3], pd[4], pd[5], pd[6], pd[7]);
        st_global_v8(dst + 32, pd[8], pd[9], pd[10], pd[11], pd[12], pd[13], pd[14], pd[15]);
      }
      tmem_st_wait();
      trace_stamp(tr, 1 + group, ntr);  // stored
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[group]);
    }
    if (ok && n_it > 0) ok = mbar_wait(acc_done, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 16);
    if (ok) {
      tc_fence_after();
      constexpr int W = HD * 4 / C::EW;  // columns of dV / dK per warp
      const int cw = (group * 2 + half) * W;
      uint16_t* dvrow = (uint16_t*)args.dV + (long long)b * args.dv_sb + (long long)kvrow * args.dv_ss +
                        (long long)h * args.dv_sh + cw;
      uint16_t* dkrow = (uint16_t*)args.dK + (long long)b * args.dk_sb + (long long)kvrow * args.dk_ss +
                        (long long)h * args.dk_sh + cw;
      uint32_t ra[W], rb[W];
      float v[W];
      if (n_it > 0) {
        if constexpr (W == 32) {
          tmem_ld32(lane_addr + C::COL_ACC0 + cw, ra);
          tmem_ld32(lane_addr + C::COL_ACC1 + cw, rb);
        } else {
          tmem_ld16(lane_addr + C::COL_ACC0 + cw, ra);
          tmem_ld16(lane_addr + C::COL_ACC1 + cw, rb);
        }
        tmem_ld_wait();
      }
#pragma unroll
      for (int i = 0; i < W; i++) v[i] = n_it > 0 ? __uint_as_float(ra[i]) : 0.f;
      if (!row_dead) store_row16_lim<W>(dvrow, v, BF, args.D - cw);
#pragma unroll
      for (int i = 0; i < W; i++) v[i] = n_it > 0 ? __uint_as_float(rb[i]) : 0.f;
      if (!row_dead) store_row16_lim<W>(dkrow, v, BF, args.D - cw);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// dQ: one CTA per 128-row query tile; streams 64-row key sub-tiles.
template <int HD, bool BF, bool DUAL>
__global__ void __launch_bounds__(BwdCfg<HD, DUAL>::THREADS, BwdCfg<HD, DUAL>::CTAS_PER_SM)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const AttnArgs args) {
  using C = BwdCfg<HD, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::TILE_BYTES;
  uint8_t* ring = sdO + C::TILE_BYTES;  // [NS] x {K sub-tile, V sub-tile}
  uint64_t* bars = (uint64_t*)(ring + C::NS * 2 * C::SUB_BYTES + C::STAT_BYTES);
  uint64_t* q_full = bars;                  // 1
  uint64_t* kv_full = bars + 1;             // NS
  uint64_t* kv_empty = kv_full + C::NS;     // NS
  uint64_t* sdp_full = kv_empty + C::NS;    // 2
  uint64_t* p_full = sdp_full + 2;          // 2
  uint64_t* acc_done = p_full + 2;          // 1
  uint64_t* a_ready = acc_done + 1;         // 1: Q and dO copied into TMEM
  uint32_t* tmem_slot = (uint32_t*)(a_ready + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (args.Sq + BQ - 1) / BQ;
  const int q_tile = args.causal ? (num_q_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * BQ;
  int n_sub = (args.Sk + BSUB - 1) / BSUB;
  if (args.causal) n_sub = min(n_sub, (q_tile + 1) * (BQ / BSUB));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::NS; i++) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; i++) { mbar_init(&sdp_full[i], 1); mbar_init(&p_full[i], 8); }
    mbar_init(acc_done, 1);
    mbar_init(a_ready, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::CH; c++) {
        tma_load_4d(sQ + c * 128 * 128, &tmQ, q_full, c * 64, q0, h, b);
        tma_load_4d(sdO + c * 128 * 128, &tmdO, q_full, c * 64, q0, h, b);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_sub; j++) {
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 21)) break;
        mbar_expect_tx(&kv_full[st], 2 * C::SUB_BYTES);
        uint8_t* sK = ring + st * 2 * C::SUB_BYTES;
        uint8_t* sV = sK + C::SUB_BYTES;
#pragma unroll
        for (int c = 0; c < C::CH; c++) {
          tma_load_4d(sK + c * BSUB * 128, &tmK, &kv_full[st], c * 64, j * BSUB, h, b);
          tma_load_4d(sV + c * BSUB * 128, &tmV, &kv_full[st], c * 64, j * BSUB, h, b);
        }
        if (++st == C::NS) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t fmt = BF ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(1u, fmt, false, false, 128, BSUB);
      const uint32_t idesc_acc = make_idesc(1u, fmt, false, true, 128, HD);
      const uint32_t qa = smem_u32(sQ), ga = smem_u32(sdO);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 22);
      if (ok && C::Q_IN_TMEM) {
        ok = mbar_wait(a_ready, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 28);
        tc_fence_after();
      }
      int st_s = 0;
      uint32_t ph_s = 0;
      auto issue_sdp = [&](int j) {
        if (!mbar_wait(&kv_full[st_s], ph_s, abort_flag, args.status, ST_ATTN_TIMEOUT, 23)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(ring + st_s * 2 * C::SUB_BYTES), va = ka + C::SUB_BYTES;
        const uint32_t d = tmem_base + (j % C::NBUF) * 128;
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          if (C::Q_IN_TMEM) {
            tc_mma_f16_ts(d, tmem_base + C::COL_QT + k * 8, kdesc_sub(ka, k), idesc_s, k != 0);       // S = Q K^T
            tc_mma_f16_ts(d + 64, tmem_base + C::COL_GT + k * 8, kdesc_sub(va, k), idesc_s, k != 0);  // dP = dO V^T
          } else {
            tc_mma_f16(d, kdesc(qa, k), kdesc_sub(ka, k), idesc_s, k != 0);
            tc_mma_f16(d + 64, kdesc(ga, k), kdesc_sub(va, k), idesc_s, k != 0);
          }
        }
        tc_commit(&sdp_full[j % C::NBUF]);
        if (++st_s == C::NS) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      if (ok && n_sub > 0) ok = issue_sdp(0);
      int st = 0;
      for (int j = 0; j < n_sub && ok; j++) {
        if (C::NBUF == 2 && j + 1 < n_sub) {
          ok = issue_sdp(j + 1);
          if (!ok) break;
        }
        const int bb = j % C::NBUF;
        ok = mbar_wait(&p_full[bb], (j / C::NBUF) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 24);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ka = smem_u32(ring + st * 2 * C::SUB_BYTES);
        const uint32_t pt = tmem_base + bb * 128 + 64;
#pragma unroll
        for (int k = 0; k < BSUB / 16; k++)  // dQ += dS K
          tc_mma_f16_ts(tmem_base + C::COL_ACC0, pt + (k >> 1) * 32 + (k & 1) * 8, mndesc_sub(ka, k), idesc_acc,
                        (j | k) != 0);
        tc_commit(&kv_empty[st]);
        if (j == n_sub - 1) tc_commit(acc_done);
        if (++st == C::NS) st = 0;
        if (C::NBUF == 1 && j + 1 < n_sub) ok = issue_sdp(j + 1);
      }
    }
    __syncwarp();
  } else {
    const int e = warp - 2;
    const int group = e >> 3;
    const int half = (e >> 2) & 1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qrow = q0 + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t my = lane_addr + group * 128 + half * 32;
    float lse2 = INFINITY, dls = 0.f;
    if (qrow < args.Sq) {
      lse2 = args.LSE[((long long)b * args.H + h) * args.Sq + qrow] * 1.4426950408889634f;
      dls = args.Delta[((long long)b * args.H + h) * args.Sq + qrow] * args.scale;
      if (lse2 == -INFINITY) lse2 = INFINITY;
    }
    bool ok = true;
    if (C::Q_IN_TMEM && group == 0) {
      // the eight warps of group 0 copy Q (half 0) and dO (half 1) into TMEM once
      ok = mbar_wait(q_full, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 29);
      if (ok) {
        tile_row_to_tmem<HD>(half == 0 ? sQ : sdO, r, lane_addr, half == 0 ? C::COL_QT : C::COL_GT);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
      }
    }
    for (int j = group; j < n_sub; j += C::NBUF) {
      ok = mbar_wait(&sdp_full[group], (j / C::NBUF) & 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 25);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BSUB + half * 32;  // first key column of this thread
      // per warp: 32 query rows (from q0 + 32 * quarter) against 32 key columns (from kv0)
      const int row0 = q0 + quarter * 32;
      const bool all_masked = args.causal && kv0 > row0 + 31;
      const bool need_mask = (args.causal && kv0 + 31 > row0) || (kv0 + 32 > args.Sk);
      uint32_t rs[32], rd[32];
      if (all_masked) {
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; i++) z[i] = 0u;
        tmem_st16(my + 64, z);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[group]);
        continue;
      }
      tmem_ld32(my, rs);
      tmem_ld32(my + 64, rd);
      tmem_ld_wait();
      uint32_t pd[16];
      auto body = [&](auto use_mask) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
          float dv[2];
#pragma unroll
          for (int u = 0; u < 2; u++) {
            const int c = 2 * i + u;
            const float e = fmaf(__uint_as_float(rs[c]), args.scale_log2, -lse2);
            float p = (HD == 64 && (c & 3) == 3 && !decltype(use_mask)::value) ? exp2_poly(e) : exp2f(e);
            if (decltype(use_mask)::value) {
              if (kv0 + c >= args.Sk || (args.causal && kv0 + c > qrow)) p = 0.f;
            }
            dv[u] = p * fmaf(__uint_as_float(rd[c]), args.scale, -dls);
          }
          pd[i] = pack16t<BF>(dv[0], dv[1]);
        }
      };
      if (need_mask) body(std::true_type{});
      else body(std::false_type{});
      tmem_st16(my + 64, pd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[group]);
    }
    if (ok && n_sub > 0) ok = mbar_wait(acc_done, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 26);
    if (ok) {
      tc_fence_after();
      constexpr int W = HD * 4 / C::EW;
      const int cw = (group * 2 + half) * W;
      const bool row_ok = qrow < args.Sq;
      uint16_t* dqrow = (uint16_t*)args.dQ + (long long)b * args.dq_sb + (long long)qrow * args.dq_ss +
                        (long long)h * args.dq_sh + cw;
      uint32_t rr[W];
      float v[W];
      if (n_sub > 0) {
        if constexpr (W == 32) tmem_ld32(lane_addr + C::COL_ACC0 + cw, rr);
        else tmem_ld16(lane_addr + C::COL_ACC0 + cw, rr);
        tmem_ld_wait();
      }
#pragma unroll
      for (int i = 0; i < W; i++) v[i] = n_sub > 0 ? __uint_as_float(rr[i]) : 0.f;
      if (row_ok) store_row16_lim<W>(dqrow, v, BF, args.D - cw);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// dQ from the spilled dS^T: dQ[q, :] = sum over keys of dS^T[key, q] * K[key, :].  One CTA per
// 128-query tile streams 64-key slices: the dS^T slice (64 keys x 128 queries, two 64-query
// chunks) is the M-major A operand, the K slice (64 keys x HD) the N-major B operand, both
// straight from TMA-written shared memory; the accumulator is HD fp32 columns of TMEM.
// 192 threads: warp 0 TMA, warp 1 MMA, warps 2-5 the epilogue (one query row per thread).
template <int HD>
struct DqDsCfg {
  static constexpr int CH = HD / 64;
  static constexpr int DS_BYTES = 2 * BSUB * 128;        // two 64-query chunks of 64 key rows
  static constexpr int K_BYTES = CH * BSUB * 128;
  static constexpr int STAGE_BYTES = DS_BYTES + K_BYTES;
  static constexpr int NS = 4;
  static constexpr int SMEM_BYTES = NS * STAGE_BYTES + 1024 + 256;
  static constexpr int THREADS = 192;
};

template <int HD, bool BF>
__global__ void __launch_bounds__(DqDsCfg<HD>::THREADS, 2)
fa_bwd_dq_ds_kernel(const __grid_constant__ CUtensorMap tmDS, const __grid_constant__ CUtensorMap tmK,
                    const AttnArgs args) {
  using C = DqDsCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;
  uint64_t* bars = (uint64_t*)(ring + C::NS * C::STAGE_BYTES);
  uint64_t* full = bars;                 // NS
  uint64_t* empty = full + C::NS;        // NS
  uint64_t* acc_done = empty + C::NS;    // 1
  uint32_t* tmem_slot = (uint32_t*)(acc_done + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (args.Sq + BQ - 1) / BQ;
  const int q_tile = args.causal ? (num_q_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * BQ;
  int n_sub = (args.Sk + BSUB - 1) / BSUB;
  if (args.causal) n_sub = min(n_sub, (q_tile + 1) * (BQ / BSUB));

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::NS; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmDS);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, HD); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_sub; j++) {
        if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, args.status, ST_ATTN_TIMEOUT, 31)) break;
        mbar_expect_tx(&full[st], C::STAGE_BYTES);
        uint8_t* sD = ring + st * C::STAGE_BYTES;
        uint8_t* sK = sD + C::DS_BYTES;
        tma_load_4d(sD, &tmDS, &full[st], q0, j * BSUB, b * args.H + h, 0);
        tma_load_4d(sD + BSUB * 128, &tmDS, &full[st], q0 + 64, j * BSUB, b * args.H + h, 0);
#pragma unroll
        for (int c = 0; c < C::CH; c++)
          tma_load_4d(sK + c * BSUB * 128, &tmK, &full[st], c * 64, j * BSUB, h, b);
        if (++st == C::NS) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1u, BF ? 1u : 0u, true, true, 128, HD);
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_sub; j++) {
        if (!mbar_wait(&full[st], ph, abort_flag, args.status, ST_ATTN_TIMEOUT, 32)) break;
        tc_fence_after();
        const uint32_t da = smem_u32(ring + st * C::STAGE_BYTES), ka = da + C::DS_BYTES;
#pragma unroll
        for (int k = 0; k < BSUB / 16; k++)
          tc_mma_f16(tmem_base, mndesc_sub(da, k), mndesc_sub(ka, k), idesc, (j | k) != 0);
        tc_commit(&empty[st]);
        if (j == n_sub - 1) tc_commit(acc_done);
        if (++st == C::NS) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qrow = q0 + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    if (n_sub > 0) ok = mbar_wait(acc_done, 0, abort_flag, args.status, ST_ATTN_TIMEOUT, 33);
    if (ok) {
      tc_fence_after();
      uint16_t* dqrow = (uint16_t*)args.dQ + (long long)b * args.dq_sb + (long long)qrow * args.dq_ss +
                        (long long)h * args.dq_sh;
#pragma unroll
      for (int c = 0; c < HD / 32; c++) {
        uint32_t rr[32];
        float v[32];
        if (n_sub > 0) {
          tmem_ld32(lane_addr + c * 32, rr);
          tmem_ld_wait();
        }
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = n_sub > 0 ? __uint_as_float(rr[i]) : 0.f;
        if (qrow < args.Sq) store_row16_lim<32>(dqrow + c * 32, v, BF, args.D - c * 32);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, HD); }
}

int make_qkv_map(CUtensorMap* m, const void* p, int in_bf16, int B, int H, int S, int D,
                 long long sb, long long ss, long long sh, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)H, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)ss * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return gbh::encode_tmap(m, in_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          4, p, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int HD, bool BF>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const AttnArgs& a, cudaStream_t s) {
  using C = FwdCfg<HD>;
  static bool configured = false;
  if (!configured) {
    GB_CUDA_OK(cudaFuncSetAttribute(fa_fwd_kernel<HD, BF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    C::SMEM_BYTES));
    configured = true;
  }
  dim3 grid((a.Sq + BQ - 1) / BQ, a.H, a.B);
  fa_fwd_kernel<HD, BF><<<grid, kFwdThreads, C::SMEM_BYTES, s>>>(tq, tk, tv, a);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

struct BwdMaps {
  CUtensorMap q128, k128, v128, g128;  // 128-row boxes (resident tiles)
  CUtensorMap q64, k64, v64, g64;      // 64-row boxes (streamed sub-tiles)
  CUtensorMap ds;                      // the dS^T spill: (query, key, batch*head), boxes of 64 x 64
};

int g_fa_dual = 1;

template <int HD, bool BF, bool DUAL>
int launch_bwd(const BwdMaps& m, const AttnArgs& a, cudaStream_t s) {
  using C = BwdCfg<HD, DUAL>;
  static bool configured = false;
  if (!configured) {
    GB_CUDA_OK(cudaFuncSetAttribute(fa_bwd_dkv_kernel<HD, BF, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    GB_CUDA_OK(cudaFuncSetAttribute(fa_bwd_dq_kernel<HD, BF, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  dim3 gkv((a.Sk + BKV - 1) / BKV, a.H, a.B);
  fa_bwd_dkv_kernel<HD, BF, DUAL><<<gkv, C::THREADS, C::SMEM_BYTES, s>>>(m.q64, m.k128, m.v128, m.g64, a);
  GB_CUDA_OK(cudaGetLastError());
  dim3 gq((a.Sq + BQ - 1) / BQ, a.H, a.B);
  if (a.dS) {
    using D = DqDsCfg<HD>;
    static bool configured_ds = false;
    if (!configured_ds) {
      GB_CUDA_OK(cudaFuncSetAttribute(fa_bwd_dq_ds_kernel<HD, BF>, cudaFuncAttributeMaxDynamicSharedMemorySize, D::SMEM_BYTES));
      configured_ds = true;
    }
    fa_bwd_dq_ds_kernel<HD, BF><<<gq, D::THREADS, D::SMEM_BYTES, s>>>(m.ds, m.k64, a);
  } else {
    fa_bwd_dq_kernel<HD, BF, DUAL><<<gq, C::THREADS, C::SMEM_BYTES, s>>>(m.q128, m.k64, m.v64, m.g128, a);
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

long long* g_trace = nullptr;

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1 };

// Timeline tracing of the dK/dV kernel (builds with -DGB_FA_TRACE only): `buf` is a device buffer of
// 3 * 512 int64 (zeroed by the caller) that CTA (0,0,0) fills with SM clock stamps; null switches it off.
// head_dim 64 backward: 1 = two CTAs per SM with one S/dP buffer each, 0 = one CTA per SM
// with two buffers and sixteen elementwise warps.
GB_EXPORT int gb_flash_tune(int dual) {
  g_fa_dual = dual;
  return 0;
}

GB_EXPORT int gb_flash_trace(long long* buf) {
  g_trace = buf;
  return 0;
}

// Forward.  q/k/v/o: 16-bit tensors addressed as [b][s][h][d] through element
// strides (sb, ss, sh) with d contiguous; head_dim a multiple of 8 up to 128.  lse (fp32,
// [B,H,Sq], natural log of the scaled scores' softmax denominator) may be null.
GB_EXPORT int gb_flash_fwd(int dtype, const void* q, const void* k, const void* v, void* o,
                           float* lse, int B, int H, int Sq, int Sk, int D, long long q_sb,
                           long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                           long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                           long long o_sb, long long o_ss, long long o_sh, float scale, int causal,
                           void* stream) {
  if (D < 8 || D > 128 || (D & 7)) {
    gbh::set_error("gb_flash_fwd: head_dim must be a multiple of 8 up to 128 (got %d)", D);
    return gbh::E_BAD_ARG;
  }
  if (causal && Sq != Sk) {
    gbh::set_error("gb_flash_fwd: causal attention needs Sq == Sk");
    return gbh::E_BAD_ARG;
  }
  if ((o_sb | o_ss | o_sh) & 7 || ((uintptr_t)o & 15)) {
    gbh::set_error("gb_flash_fwd: output strides must be multiples of 8 elements");
    return gbh::E_BAD_ARG;
  }
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.B = B; a.H = H; a.Sq = Sq; a.Sk = Sk; a.D = D;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal; a.in_bf16 = dtype == DT_BF16;
  a.O = o; a.LSE = lse; a.o_sb = o_sb; a.o_ss = o_ss; a.o_sh = o_sh;
  a.status = gbh::status_ptr();
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_qkv_map(&tq, q, a.in_bf16, B, H, Sq, D, q_sb, q_ss, q_sh, BQ))) return rc;
  if ((rc = make_qkv_map(&tk, k, a.in_bf16, B, H, Sk, D, k_sb, k_ss, k_sh, BKF))) return rc;
  if ((rc = make_qkv_map(&tv, v, a.in_bf16, B, H, Sk, D, v_sb, v_ss, v_sh, BKF))) return rc;
  // head sizes other than 64 / 128 run the next larger kernel: the tensor maps describe the real
  // extent, loads beyond it are zero-filled by TMA, stores stop at the real extent
  if (D > 64)
    return a.in_bf16 ? launch_fwd<128, true>(tq, tk, tv, a, (cudaStream_t)stream)
                     : launch_fwd<128, false>(tq, tk, tv, a, (cudaStream_t)stream);
  return a.in_bf16 ? launch_fwd<64, true>(tq, tk, tv, a, (cudaStream_t)stream)
                   : launch_fwd<64, false>(tq, tk, tv, a, (cudaStream_t)stream);
}

GB_EXPORT int gb_flash_delta(int dtype, const void* o, const void* dout, float* delta, int B, int H,
                             int S, int D, long long o_sb, long long o_ss, long long o_sh,
                             long long g_sb, long long g_ss, long long g_sh, void* stream) {
  long long total = (long long)B * H * S;
  if (total < 1) return gbh::E_OK;
  const bool vec = (D == 64 || D == 128) && !((o_sb | o_ss | o_sh | g_sb | g_ss | g_sh) & 7) &&
                   !(((uintptr_t)o | (uintptr_t)dout) & 15);
  if (vec) {
    const int tpr = D / 8, rpb = 256 / tpr;
    int grid = (int)((total + rpb - 1) / rpb < 148 * 8 ? (total + rpb - 1) / rpb : 148 * 8);
    cudaStream_t st = (cudaStream_t)stream;
#define GB_DELTA(T, TPR)                                                                               \
  fa_delta_vec_kernel<T, TPR><<<grid, 256, 0, st>>>((const T*)o, (const T*)dout, delta, B, H, S, o_sb, \
                                                    o_ss, o_sh, g_sb, g_ss, g_sh)
    if (dtype == DT_BF16) { if (D == 64) GB_DELTA(__nv_bfloat16, 8); else GB_DELTA(__nv_bfloat16, 16); }
    else { if (D == 64) GB_DELTA(__half, 8); else GB_DELTA(__half, 16); }
#undef GB_DELTA
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  int grid = (int)((total + 7) / 8 < 148 * 16 ? (total + 7) / 8 : 148 * 16);
  if (dtype == DT_BF16)
    fa_delta_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, H, S, D, o_sb, o_ss, o_sh, g_sb, g_ss, g_sh);
  else
    fa_delta_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __half*)o, (const __half*)dout, delta, B, H, S, D, o_sb, o_ss, o_sh, g_sb, g_ss, g_sh);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Backward.  All tensors are [b][s][h][d] through element strides, d contiguous.
// lse: the forward's output; delta: from gb_flash_delta.  Writes dq, dk, dv.
// Bytes of workspace with which gb_flash_bwd_ws computes dQ from a spilled dS^T.
GB_EXPORT long long gb_flash_bwd_ws_bytes(int B, int H, int Sq, int Sk) {
  const long long ld = (Sq + 127) / 128 * 128, rows = (Sk + 127) / 128 * 128;
  return (long long)B * H * rows * ld * 2;
}

GB_EXPORT int gb_flash_bwd_ws(int dtype, const void* q, const void* k, const void* v, const void* dout,
                              const float* lse, const float* delta, void* dq, void* dk, void* dv,
                              int B, int H, int Sq, int Sk, int D, const long long* strides,
                              float scale, int causal, void* ws, long long ws_bytes, void* stream);

GB_EXPORT int gb_flash_bwd(int dtype, const void* q, const void* k, const void* v, const void* dout,
                           const float* lse, const float* delta, void* dq, void* dk, void* dv,
                           int B, int H, int Sq, int Sk, int D, const long long* strides,
                           float scale, int causal, void* stream) {
  return gb_flash_bwd_ws(dtype, q, k, v, dout, lse, delta, dq, dk, dv, B, H, Sq, Sk, D, strides, scale, causal,
                         nullptr, 0, stream);
}

// The same with an optional workspace (32-byte aligned, gb_flash_bwd_ws_bytes bytes, contents
// arbitrary).  With it the dK/dV kernel also writes dS^T and dQ is one product dS K read back
// from it; without it (null, or too small) a second kernel recomputes the scores for dQ.
GB_EXPORT int gb_flash_bwd_ws(int dtype, const void* q, const void* k, const void* v, const void* dout,
                              const float* lse, const float* delta, void* dq, void* dk, void* dv,
                              int B, int H, int Sq, int Sk, int D, const long long* strides,
                              float scale, int causal, void* ws, long long ws_bytes, void* stream) {
  // strides: 7 triples (sb, ss, sh) for q, k, v, dout, dq, dk, dv
  if (D < 8 || D > 128 || (D & 7)) {
    gbh::set_error("gb_flash_bwd: head_dim must be a multiple of 8 up to 128 (got %d)", D);
    return gbh::E_BAD_ARG;
  }
  if (causal && Sq != Sk) {
    gbh::set_error("gb_flash_bwd: causal attention needs Sq == Sk");
    return gbh::E_BAD_ARG;
  }
  for (int i = 12; i < 21; i++)
    if (strides[i] & 7) {
      gbh::set_error("gb_flash_bwd: gradient strides must be multiples of 8 elements");
      return gbh::E_BAD_ARG;
    }
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.B = B; a.H = H; a.Sq = Sq; a.Sk = Sk; a.D = D;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal; a.in_bf16 = dtype == DT_BF16;
  a.LSE = const_cast<float*>(lse); a.Delta = delta;
  a.dQ = dq; a.dK = dk; a.dV = dv;
  a.dq_sb = strides[12]; a.dq_ss = strides[13]; a.dq_sh = strides[14];
  a.dk_sb = strides[15]; a.dk_ss = strides[16]; a.dk_sh = strides[17];
  a.dv_sb = strides[18]; a.dv_ss = strides[19]; a.dv_sh = strides[20];
  a.status = gbh::status_ptr();
  a.trace = g_trace;
  BwdMaps m;
  int rc;
  if ((rc = make_qkv_map(&m.q128, q, a.in_bf16, B, H, Sq, D, strides[0], strides[1], strides[2], 128))) return rc;
  if ((rc = make_qkv_map(&m.k128, k, a.in_bf16, B, H, Sk, D, strides[3], strides[4], strides[5], 128))) return rc;
  if ((rc = make_qkv_map(&m.v128, v, a.in_bf16, B, H, Sk, D, strides[6], strides[7], strides[8], 128))) return rc;
  if ((rc = make_qkv_map(&m.g128, dout, a.in_bf16, B, H, Sq, D, strides[9], strides[10], strides[11], 128))) return rc;
  if ((rc = make_qkv_map(&m.q64, q, a.in_bf16, B, H, Sq, D, strides[0], strides[1], strides[2], 64))) return rc;
  if ((rc = make_qkv_map(&m.k64, k, a.in_bf16, B, H, Sk, D, strides[3], strides[4], strides[5], 64))) return rc;
  if ((rc = make_qkv_map(&m.v64, v, a.in_bf16, B, H, Sk, D, strides[6], strides[7], strides[8], 64))) return rc;
  if ((rc = make_qkv_map(&m.g64, dout, a.in_bf16, B, H, Sq, D, strides[9], strides[10], strides[11], 64))) return rc;
  // (the kernel addresses the spill with 32-bit byte offsets: at most 4 GiB)
  if (ws != nullptr && ws_bytes >= gb_flash_bwd_ws_bytes(B, H, Sq, Sk) && !((uintptr_t)ws & 31) &&
      gb_flash_bwd_ws_bytes(B, H, Sq, Sk) <= (1LL << 32)) {
    a.dS = ws;
    a.ds_ld = (Sq + 127) / 128 * 128;
    a.ds_rows = (Sk + 127) / 128 * 128;
    uint64_t dims[4] = {(uint64_t)a.ds_ld, (uint64_t)a.ds_rows, (uint64_t)B * H, 1};
    uint64_t st[3] = {(uint64_t)a.ds_ld * 2, (uint64_t)a.ds_ld * a.ds_rows * 2, (uint64_t)a.ds_ld * a.ds_rows * 2 * B * H};
    uint32_t box[4] = {64, 64, 1, 1};
    if ((rc = gbh::encode_tmap(&m.ds, a.in_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                               4, ws, dims, st, box, CU_TENSOR_MAP_SWIZZLE_128B)))
      return rc;
  }
  if (D > 64)
    return a.in_bf16 ? launch_bwd<128, true, false>(m, a, (cudaStream_t)stream)
                     : launch_bwd<128, false, false>(m, a, (cudaStream_t)stream);
  if (g_fa_dual)
    return a.in_bf16 ? launch_bwd<64, true, true>(m, a, (cudaStream_t)stream)
                     : launch_bwd<64, false, true>(m, a, (cudaStream_t)stream);
  return a.in_bf16 ? launch_bwd<64, true, false>(m, a, (cudaStream_t)stream)
                   : launch_bwd<64, false, false>(m, a, (cudaStream_t)stream);
}
