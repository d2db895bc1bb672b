// Implicit-GEMM convolution on tcgen05: forward, data gradient and weight gradient without an
// im2col matrix in memory.
//
// The reference computes a convolution as a dense 0/1 gather-matrix product that materialises
// the (N, L, C*T) column tensor, then a batched MatMul (nn/conv.go:341-380, nn/gather.go:99-181),
// and lets autograd differentiate those tape nodes.  Here the column tensor never exists: the
// producer warps of each CTA gather the operand tiles straight from the (N, C, spatial) tensors
// into the 128-byte-swizzled shared-memory layout that tcgen05.mma reads (through the same
// int32 window index map the pooling and fold kernels use: entry [l][tap] is the source position
// of tap `tap` of output position `l`, or -1 for padding), one elected thread issues the MMAs into
// a 128 x 128 fp32 accumulator in tensor memory, and the same warps run the epilogue.
//
//   forward   y[n][co][l]  = bias[co] + sum_{c,tap} W[co][c][tap] * x[n][c][idx[l][tap]]
//             GEMM per image: M = C_out, N = L, K = C_in * T; A = weights, B = gathered windows.
//   dgrad     the same kernel with x := dy, idx := the inverse map ([s][tap] -> l or -1) and the
//             weights regrouped as a (C_in, C_out * T) matrix.
//   wgrad     dW[co][(c,tap)] = sum_{n,l} dy[n][co][l] * x[n][c][idx[l][tap]]
//             ONE GEMM over the whole batch: M = C_out, N = C_in * T, K = N_img * L, split over
//             CTAs along K into fp32 partials that a second kernel adds in split order
//             (deterministic).
//
// No tensor map is involved (every operand is gathered with ordinary loads from this GPU's own
// memory), so the kernels may run inside multi-GPU jobs.  Every wait is bounded.
#include "common.cuh"

using namespace gb;

namespace {

constexpr int CBM = 128, CBN = 128, CBK = 64, CSTAGES = 2;
constexpr int CA_BYTES = CBM * CBK * 2, CB_BYTES = CBN * CBK * 2, CSTAGE_BYTES = CA_BYTES + CB_BYTES;
constexpr int CPRODUCERS = 256;            // threads 0..127 fill A rows, 128..255 fill B rows
constexpr int CTHREADS = CPRODUCERS + 32;  // + the MMA warp
constexpr int CMAX_T_SMEM = 32;            // window taps up to which the forward stages its index rows
constexpr int CSMEM = CSTAGES * CSTAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + CBN * CMAX_T_SMEM * 4;

struct ConvArgs {
  // forward / dgrad
  const uint16_t* W;       // (M, K) row-major weights, K = C * T ordered (c, tap)
  int w_vec;               // rows may be read in 16-byte pieces (K % 8 == 0 and an aligned base)
  const int2* ktab;        // [K rounded up to 128]: {c * S, tap} for k < K, {-1, 0} beyond
  const uint16_t* X;       // (Nimg, C, S): the tensor whose windows are gathered
  const int* idx;          // [L][T]
  void* Y;                 // forward / dgrad: (Nimg, M, L) 16-bit; wgrad: fp32 partials [splits][M][KK]
  const uint16_t* bias;    // [M], same 16-bit type, or null
  // wgrad
  const uint16_t* DY;      // (Nimg, M, L)
  int Nimg, C, S, L, T, M;
  int bf16;
  long long r_per_split;   // wgrad: contraction indices per split (multiple of 64)
  int* status;
};

__device__ __forceinline__ float raw16_to_float(uint16_t u, int bf) {
  return bf ? __uint_as_float((uint32_t)u << 16) : __half2float(__ushort_as_half(u));
}

// One 16-byte chunk (8 consecutive k) into row `row`, chunk `c8` of a K-major 128-byte-swizzled tile.
__device__ __forceinline__ void store_chunk(uint8_t* tile, int row, int c8, const uint16_t (&v)[8]) {
  uint4 u;
  u.x = (uint32_t)v[0] | ((uint32_t)v[1] << 16);
  u.y = (uint32_t)v[2] | ((uint32_t)v[3] << 16);
  u.z = (uint32_t)v[4] | ((uint32_t)v[5] << 16);
  u.w = (uint32_t)v[6] | ((uint32_t)v[7] << 16);
  *reinterpret_cast<uint4*>(tile + row * 128 + ((c8 ^ (row & 7)) << 4)) = u;
}

// MODE 0: forward / dgrad (grid: L tiles, M tiles, images); MODE 1: wgrad (grid: KK tiles, M tiles, splits)
template <int MODE>
__global__ void __launch_bounds__(CTHREADS, 2)
conv_igemm_kernel(const ConvArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + CSTAGES * CSTAGE_BYTES);
  uint64_t* full_bar = bars;              // [CSTAGES], 8 arrivals: one per producer warp
  uint64_t* empty_bar = bars + CSTAGES;   // [CSTAGES], 1 arrival: tcgen05.commit
  uint64_t* done_bar = bars + 2 * CSTAGES;
  uint32_t* tmem_slot = (uint32_t*)(done_bar + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = a.C * a.T;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CSTAGES; s++) { mbar_init(&full_bar[s], CPRODUCERS / 32); mbar_init(&empty_bar[s], 1); }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, CBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // contraction range of this CTA, in k-blocks of 64
  long long kc_begin, kc_end;   // element indices along the contraction
  if (MODE == 0) {
    kc_begin = 0;
    kc_end = K;
  } else {
    const long long R = (long long)a.Nimg * a.L;
    kc_begin = (long long)blockIdx.z * a.r_per_split;
    kc_end = kc_begin + a.r_per_split < R ? kc_begin + a.r_per_split : R;
  }
  const int nkb = kc_end > kc_begin ? (int)((kc_end - kc_begin + CBK - 1) / CBK) : 0;
  const int m0 = blockIdx.y * CBM, n0 = blockIdx.x * CBN;

  if (warp < 8) {
    // ---------------- producers ----------------
    // Warps 0-3 fill the A tile, warps 4-7 the B tile, 32 rows each.  The kernel is bound by the
    // instructions of these gathers, so they are kept to a handful per element: the split of a
    // contraction index k into (channel offset, tap) comes from a table built once per geometry
    // (ktab[k] = {c * S, tap}, {-1, 0} past the end), window index rows are staged in shared
    // memory, offsets are 32-bit, and every load is unconditional (offset 0 when the element is
    // padding, the value zeroed afterwards) so that many are in flight per thread.
    const bool is_a = warp < 4;
    const int wq = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const int e0 = 2 * lane;
    int* sidx = reinterpret_cast<int*>(smem + CSTAGES * CSTAGE_BYTES + 256);   // [128][T] (fwd) or [64][T] (wgrad)
    // Forward / dgrad tiles run over the positions of ALL images (p = image * L + l), so a plane whose
    // size is not a multiple of the tile (13 x 13 = 169) does not leave a mostly empty second tile per image.
    const long long P = (long long)a.Nimg * a.L;
    if (MODE == 0 && !is_a) {
      // the index rows of this CTA's 128 positions, staged once
      const int total = CBN * a.T;
      for (int i = threadIdx.x - CBM; i < total; i += CBN) {
        const long long pp = (long long)n0 + i / a.T;
        sidx[i] = pp < P ? __ldg(a.idx + (pp % a.L) * a.T + i % a.T) : -1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four B warps only
    }
    for (int kb = 0; kb < nkb && ok; kb++) {
      if (lane == 0) ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, a.status, ST_CONV_TIMEOUT, 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      uint8_t* tile = smem + stage * CSTAGE_BYTES + (is_a ? 0 : CA_BYTES);
      const long long k0 = kc_begin + (long long)kb * CBK;
      if (MODE == 0 && is_a) {
        // weights as a row-major (M, K) matrix: thread = row
        const int row = threadIdx.x;
        const int m = m0 + row;
        const uint16_t* wr = a.W + (long long)(m < a.M ? m : a.M - 1) * K;
        if (a.w_vec) {
#pragma unroll
          for (int c8 = 0; c8 < 8; c8++) {
            const int k = (int)k0 + c8 * 8;
            uint4 u = make_uint4(0u, 0u, 0u, 0u);
            if (m < a.M && k < K) u = __ldg(reinterpret_cast<const uint4*>(wr + k));   // K % 8 == 0: whole chunks
            *reinterpret_cast<uint4*>(tile + row * 128 + ((c8 ^ (row & 7)) << 4)) = u;
          }
        } else {
#pragma unroll 1
          for (int h = 0; h < 4; h++) {
            uint16_t v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const int k = (int)k0 + h * 16 + j;
              v[j] = __ldg(wr + (k < K ? k : K - 1));
              if (!(m < a.M && k < K)) v[j] = 0;
            }
            store_chunk(tile, row, 2 * h, *reinterpret_cast<const uint16_t(*)[8]>(&v[0]));
            store_chunk(tile, row, 2 * h + 1, *reinterpret_cast<const uint16_t(*)[8]>(&v[8]));
          }
        }
      } else if (MODE == 0) {
        // window operand, lanes along positions: consecutive positions read consecutive elements
        const int row = wq * 32 + lane;
        const int* ir = sidx + row * a.T;
        const long long pp = (long long)n0 + row;
        const uint16_t* xn = a.X + (pp < P ? pp / a.L : 0) * a.C * a.S;   // this row's image (padding rows read image 0, zeroed)
        const int2* kt = a.ktab + k0;
#pragma unroll 1
        for (int h = 0; h < 4; h++) {
          int off[16];
          uint16_t v[16];
#pragma unroll
          for (int j = 0; j < 16; j++) {
            const int2 t = __ldg(kt + h * 16 + j);       // the same entry for the whole warp
            const int src = ir[t.y];
            off[j] = (t.x >= 0 && src >= 0) ? t.x + src : -1;
          }
#pragma unroll
          for (int j = 0; j < 16; j++) v[j] = __ldg(xn + (off[j] >= 0 ? off[j] : 0));
#pragma unroll
          for (int j = 0; j < 16; j++) v[j] = off[j] >= 0 ? v[j] : (uint16_t)0;
          store_chunk(tile, row, 2 * h, *reinterpret_cast<const uint16_t(*)[8]>(&v[0]));
          store_chunk(tile, row, 2 * h + 1, *reinterpret_cast<const uint16_t(*)[8]>(&v[8]));
        }
      } else {
        // weight gradient: lanes along the contraction index r = image * L + l
        int nn[2], ll[2];
        bool kv[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const long long r = k0 + e0 + e;
          kv[e] = r < kc_end;
          const long long rc = kv[e] ? r : kc_end - 1;
          nn[e] = (int)(rc / a.L);
          ll[e] = (int)(rc % a.L);
        }
        if (!is_a) {
          // index rows of this k-block's 64 positions: [64][T]
          asm volatile("bar.sync 1, 128;" ::: "memory");   // the previous k-block's readers are done
          const int total = CBK * a.T;
          for (int i = threadIdx.x - CBM; i < total; i += CBN) {
            const long long r = k0 + i / a.T;
            sidx[i] = r < kc_end ? __ldg(a.idx + (r % a.L) * a.T + i % a.T) : -1;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const uint16_t* b0 = is_a ? a.DY + ((long long)nn[0] * a.M) * a.L + ll[0] : a.X + (long long)nn[0] * a.C * a.S;
        const uint16_t* b1 = is_a ? a.DY + ((long long)nn[1] * a.M) * a.L + ll[1] : a.X + (long long)nn[1] * a.C * a.S;
#pragma unroll 1
        for (int rb = 0; rb < 32; rb += 8) {
          uint16_t v[8][2];
          int o0[8], o1[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int rowi = wq * 32 + rb + j;
            if (is_a) {
              const int m = m0 + rowi;
              o0[j] = o1[j] = m < a.M ? m * a.L : -1;
            } else {
              const int kk = n0 + rowi;
              const int2 t = __ldg(a.ktab + kk);           // ktab covers K rounded up to 128
              const int s0 = sidx[e0 * a.T + t.y], s1 = sidx[(e0 + 1) * a.T + t.y];
              o0[j] = (t.x >= 0 && s0 >= 0) ? t.x + s0 : -1;
              o1[j] = (t.x >= 0 && s1 >= 0) ? t.x + s1 : -1;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j++) {
            v[j][0] = __ldg(b0 + (o0[j] >= 0 ? o0[j] : 0));
            v[j][1] = __ldg(b1 + (o1[j] >= 0 ? o1[j] : 0));
          }
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int rowi = wq * 32 + rb + j;
            const uint32_t lo = (o0[j] >= 0 && kv[0]) ? v[j][0] : 0u, hi = (o1[j] >= 0 && kv[1]) ? v[j][1] : 0u;
            uint8_t* d = tile + rowi * 128 + ((((e0 >> 3) ^ (rowi & 7))) << 4) + (e0 & 7) * 2;
            *reinterpret_cast<uint32_t*>(d) = lo | (hi << 16);
          }
        }
      }
      fence_proxy_async_smem();   // generic-proxy writes become visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[stage]);
      if (++stage == CSTAGES) { stage = 0; phase ^= 1; }
    }
  } else if (elect_one()) {
    // ---------------- MMA issuer (one thread) ----------------
    uint32_t id = make_idesc(1u, 0u, false, false, CBM, CBN);
    if (a.bf16) id |= (1u << 7) | (1u << 10);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; kb++) {
      ok = mbar_wait(&full_bar[stage], phase, abort_flag, a.status, ST_CONV_TIMEOUT, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = smem_u32(smem + stage * CSTAGE_BYTES);
      const uint32_t sb = sa + CA_BYTES;
#pragma unroll
      for (int k = 0; k < CBK / 16; k++) {
        // K-major tiles: 8-row groups 1024 B apart, one MMA step is 32 B along K
        tc_mma_f16(tmem_base, make_smem_desc_sw128(sa + k * 32, 16, 1024), make_smem_desc_sw128(sb + k * 32, 16, 1024),
                   id, (kb > 0) || k != 0);
      }
      tc_commit(&empty_bar[stage]);
      if (++stage == CSTAGES) { stage = 0; phase ^= 1; }
    }
    tc_commit(done_bar);   // arrives when every MMA above has finished (at once if there were none)
  }

  // ---------------- epilogue: the eight producer warps ----------------
  // tcgen05.ld gives a thread one accumulator row (lane = row).  Rows of the outputs are far
  // apart in memory, so each warp turns its 32 x 32 block around through shared memory (the
  // ring is idle by now) and stores with lanes along the contiguous dimension.
  if (warp < 8) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(done_bar, 0, abort_flag, a.status, ST_CONV_TIMEOUT, 3);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (ok) {
      tc_fence_after();
      const int q = warp & 3, half = warp >> 2;        // TMEM lane quarter, column half
      const int mrow0 = m0 + q * 32;
      float* stf = reinterpret_cast<float*>(smem + warp * (32 * 33 * 4));   // [32][33] floats per warp
#pragma unroll 1
      for (int cc = 0; cc < 2; cc++) {
        const int col0 = half * 64 + cc * 32;
        uint32_t r[32];
        if (nkb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + col0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = 0u;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j++) stf[lane * 33 + j] = __uint_as_float(r[j]);
        __syncwarp();
        const int col = n0 + col0 + lane;
        if (MODE == 0) {
          const long long pp = (long long)n0 + col0 + lane;          // position over all images
          const bool live = pp < (long long)a.Nimg * a.L;
          const long long img = live ? pp / a.L : 0;
          const int lpos = (int)(pp - img * a.L);
          uint16_t* yb = (uint16_t*)a.Y + img * a.M * a.L + lpos;
          for (int rr = 0; rr < 32; rr++) {
            const int m = mrow0 + rr;
            if (m >= a.M) break;
            if (live) {
              const float bv = a.bias ? raw16_to_float(__ldg(a.bias + m), a.bf16) : 0.f;
              const float v = stf[rr * 33 + lane] + bv;
              yb[(long long)m * a.L] =
                  a.bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
            }
          }
        } else {
          float* pb = (float*)a.Y + (long long)blockIdx.z * a.M * K;
          for (int rr = 0; rr < 32; rr++) {
            const int m = mrow0 + rr;
            if (m >= a.M) break;
            if (col < K) pb[(long long)m * K + col] = stf[rr * 33 + lane];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem_base, CBN);
}

// dW[m][kk] = (beta ? dW : 0) + sum_s part[s][m][kk], in split order; written in the 16-bit type
__global__ void conv_wgrad_finish_kernel(const float* __restrict__ part, uint16_t* __restrict__ dW, long long n,
                                         int splits, int bf16, int beta) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float s = beta ? raw16_to_float(dW[i], bf16) : 0.f;
#pragma unroll 8
    for (int sp = 0; sp < splits; sp++) s += part[(long long)sp * n + i];
    dW[i] = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(s)) : __half_as_ushort(__float2half_rn(s));
  }
}

// Forward convolution with a short contraction (C * T <= 32: the first layer of an image network,
// 3 channels x 3 x 3).  A tensor-core tile would spend its time on set-up: the implicit-GEMM kernel needs
// about 15 us per CTA whatever the contraction length.  Here a thread owns one output position of one
// image: it gathers its K inputs into registers once and then produces every output channel, four at a
// time, with packed fp32 FMAs against weights that sit in shared memory as [k][channel] (one 16-byte
// broadcast load feeds two FMA pairs).  Stores are coalesced along the positions.
constexpr int kDirectK = 32;
template <int KMAX>
__global__ void __launch_bounds__(256)
conv_direct_small_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, const int* __restrict__ idx,
                         const uint16_t* __restrict__ bias, uint16_t* __restrict__ y, int C, int S, int L, int T,
                         int M, int bf16) {
  extern __shared__ __align__(16) float sw[];          // [KMAX][M] weights, then [M] bias
  float* sbias = sw + KMAX * M;
  const int K = C * T;
  for (int i = threadIdx.x; i < KMAX * M; i += blockDim.x) {
    const int k = i / M, m = i - k * M;
    sw[i] = k < K ? raw16_to_float(__ldg(w + (long long)m * K + k), bf16) : 0.f;
  }
  for (int m = threadIdx.x; m < M; m += blockDim.x) sbias[m] = bias ? raw16_to_float(__ldg(bias + m), bf16) : 0.f;
  __syncthreads();
  const int n = blockIdx.y;
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  const uint16_t* xn = x + (long long)n * C * S;
  float v[KMAX];
  {
    int c = 0, tap = 0;
#pragma unroll
    for (int k = 0; k < KMAX; k++) {
      float f = 0.f;
      if (k < K) {
        const int src = __ldg(idx + (long long)l * T + tap);
        if (src >= 0) f = raw16_to_float(__ldg(xn + (long long)c * S + src), bf16);
        if (++tap == T) { tap = 0; c++; }
      }
      v[k] = f;
    }
  }
  uint16_t* yn = y + (long long)n * M * L + l;
  const float4* sw4 = reinterpret_cast<const float4*>(sw);
  const int M4 = M >> 2;
  for (int m4 = 0; m4 < M4; m4++) {
    float2 a0 = make_float2(sbias[4 * m4], sbias[4 * m4 + 1]);
    float2 a1 = make_float2(sbias[4 * m4 + 2], sbias[4 * m4 + 3]);
#pragma unroll
    for (int k = 0; k < KMAX; k++) {
      const float4 wv = sw4[k * M4 + m4];
      const float2 vv = make_float2(v[k], v[k]);
      a0 = __ffma2_rn(make_float2(wv.x, wv.y), vv, a0);
      a1 = __ffma2_rn(make_float2(wv.z, wv.w), vv, a1);
    }
    const float o[4] = {a0.x, a0.y, a1.x, a1.y};
#pragma unroll
    for (int j = 0; j < 4; j++)
      yn[(long long)(4 * m4 + j) * L] = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(o[j]))
                                             : __half_as_ushort(__float2half_rn(o[j]));
  }
}

// Weight gradient for the same short contractions (C * T <= 32), M = 32, 64 or 128 output channels:
//   dW[m][k] = sum over positions p (all images) of dy[p][m] * patch[p][k].
// A CTA walks its share of the positions in tiles of 256: every thread gathers the K inputs of one
// position and the M gradients of that position into shared memory (rows padded by four words so that
// 16-byte accesses of consecutive rows fall into different banks), then the CTA's 256 threads form
// 256 / M position groups of M threads; a thread accumulates a 4 (channels) x 8 (k) block of dW over its
// group's positions with three 16-byte shared loads per 32 FMAs.  The groups are added in order at the
// end and the CTA writes one partial matrix; conv_wgrad_finish_kernel adds the CTAs in index order.
template <int M>
__global__ void __launch_bounds__(256, 2)
conv_wgrad_small_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ dy, const int* __restrict__ idx,
                        float* __restrict__ part, int Nimg, int C, int S, int L, int T, int bf16) {
  constexpr int KMAX = kDirectK, PS = KMAX + 4, GS = M + 4, GROUPS = 256 / M;
  extern __shared__ __align__(16) float smw[];
  float* sP = smw;                 // [256][PS]  patches
  float* sG = smw + 256 * PS;      // [256][GS]  gradients
  const int K = C * T;
  const long long P = (long long)Nimg * L;
  const long long per = ((P + gridDim.x - 1) / gridDim.x + 255) / 256 * 256;
  const long long p_begin = (long long)blockIdx.x * per;
  const long long p_end = p_begin + per < P ? p_begin + per : P;
  const int t = threadIdx.x;
  const int grp = t / M, tm = t % M;           // position group; 4-channel block and k block inside it
  const int co4 = tm >> 2, kq = tm & 3;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
  for (long long p0 = p_begin; p0 < p_end; p0 += 256) {
    __syncthreads();                            // the previous tile has been consumed
    {
      const long long p = p0 + t;
      const bool live = p < p_end;
      const long long n = live ? p / L : 0;
      const int l = (int)(p - n * L);
      const uint16_t* xn = x + n * C * S;
      float v[KMAX];
      int c = 0, tap = 0;
#pragma unroll
      for (int k = 0; k < KMAX; k++) {
        float f = 0.f;
        if (k < K) {
          const int src = live ? __ldg(idx + (long long)l * T + tap) : -1;
          if (src >= 0) f = raw16_to_float(__ldg(xn + (long long)c * S + src), bf16);
          if (++tap == T) { tap = 0; c++; }
        }
        v[k] = f;
      }
#pragma unroll
      for (int k4 = 0; k4 < KMAX / 4; k4++)
        *reinterpret_cast<float4*>(sP + t * PS + 4 * k4) = make_float4(v[4 * k4], v[4 * k4 + 1], v[4 * k4 + 2], v[4 * k4 + 3]);
      const uint16_t* gn = dy + n * M * L + l;
#pragma unroll 4
      for (int m4 = 0; m4 < M / 4; m4++) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
          g.x = raw16_to_float(__ldg(gn + (long long)(4 * m4) * L), bf16);
          g.y = raw16_to_float(__ldg(gn + (long long)(4 * m4 + 1) * L), bf16);
          g.z = raw16_to_float(__ldg(gn + (long long)(4 * m4 + 2) * L), bf16);
          g.w = raw16_to_float(__ldg(gn + (long long)(4 * m4 + 3) * L), bf16);
        }
        *reinterpret_cast<float4*>(sG + t * GS + 4 * m4) = g;
      }
    }
    __syncthreads();
    // group grp takes positions grp, grp + GROUPS, ... of the tile
#pragma unroll 2
    for (int q = grp; q < 256; q += GROUPS) {
      const float4 g = *reinterpret_cast<const float4*>(sG + q * GS + 4 * co4);
      const float4 pa = *reinterpret_cast<const float4*>(sP + q * PS + 8 * kq);
      const float4 pb = *reinterpret_cast<const float4*>(sP + q * PS + 8 * kq + 4);
      const float gv[4] = {g.x, g.y, g.z, g.w};
      const float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(gv[i], pv[j], acc[i][j]);
    }
  }
  // add the position groups in order: group 0 writes, the others add one after another
  __syncthreads();
  float* red = smw;                             // [M][KMAX], reusing the tile memory
  for (int gsel = 0; gsel < GROUPS; gsel++) {
    if (grp == gsel) {
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float* dst = red + (4 * co4 + i) * KMAX + 8 * kq + j;
          *dst = gsel == 0 ? acc[i][j] : *dst + acc[i][j];
        }
    }
    __syncthreads();
  }
  float* out = part + (long long)blockIdx.x * M * K;
  for (int i = t; i < M * K; i += 256) out[i] = red[(i / K) * KMAX + i % K];
}

inline int wgrad_small_ctas(long long P) {
  long long g = (P + 255) / 256;
  if (g > 2 * 148) g = 2 * 148;
  return g < 1 ? 1 : (int)g;
}
inline bool wgrad_small_ok(int C, int T, int M) { return C * T <= kDirectK && (M == 32 || M == 64 || M == 128); }

int set_attr_once() {
  static bool done = false;
  if (!done) {
    GB_CUDA_OK(cudaFuncSetAttribute(conv_igemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, CSMEM));
    GB_CUDA_OK(cudaFuncSetAttribute(conv_igemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, CSMEM));
    done = true;
  }
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1 };

// y[n][m][l] = bias[m] + sum_{c,tap} W[m][c * T + tap] * x[n][c][idx[l][tap]] for 16-bit tensors.
// w: (M, C * T) row-major.  The forward passes the (C_out, C_in, T) weights as they are; the data
// gradient passes x := dy, idx := the inverse map and the weights regrouped as (C_in, C_out * T).
// ktab: gb_conv_ktab_len(C, T) int pairs {c * S, tap} ({-1, 0} past C * T), built once per geometry.
GB_EXPORT int gb_conv_ktab_len(int C, int T) { return (C * T + 127) / 128 * 128; }

GB_EXPORT int gb_conv_igemm(int dtype, const void* x, const void* w, const int* ktab, const int* idx,
                            const void* bias, void* y, int Nimg, int C, int S, int L, int T, int M, void* stream) {
  if (dtype != DT_BF16 && dtype != DT_F16) {
    gbh::set_error("gb_conv_igemm: bf16 or fp16 tensors");
    return gbh::E_BAD_ARG;
  }
  if (Nimg <= 0 || C <= 0 || L <= 0 || T <= 0 || M <= 0 || Nimg > 65535 || T > CMAX_T_SMEM ||
      (long long)C * S >= (1LL << 31) || (long long)M * L >= (1LL << 31) || (long long)Nimg * L >= (1LL << 31) - CBN) {
    gbh::set_error("gb_conv_igemm: geometry out of range (at most %d taps, 65535 images)", CMAX_T_SMEM);
    return gbh::E_BAD_ARG;
  }
  int rc = set_attr_once();
  if (rc) return rc;
  ConvArgs a;
  memset(&a, 0, sizeof(a));
  a.W = (const uint16_t*)w;
  a.w_vec = ((C * T) % 8 == 0) && (((uintptr_t)w & 15) == 0);
  a.ktab = (const int2*)ktab;
  a.X = (const uint16_t*)x; a.idx = idx; a.Y = y; a.bias = (const uint16_t*)bias;
  a.Nimg = Nimg; a.C = C; a.S = S; a.L = L; a.T = T; a.M = M;
  a.bf16 = dtype == DT_BF16;
  a.status = gbh::status_ptr();
  dim3 grid((unsigned)(((long long)Nimg * L + CBN - 1) / CBN), (M + CBM - 1) / CBM, 1);
  conv_igemm_kernel<0><<<grid, CTHREADS, CSMEM, (cudaStream_t)stream>>>(a);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Whether gb_conv_direct_small takes a forward convolution: a contraction of at most 32 and a channel
// count that is a multiple of 4 whose weights fit in 48 KB of shared memory.
GB_EXPORT int gb_conv_direct_ok(int C, int T, int M) {
  return C * T <= kDirectK && (M & 3) == 0 && M > 0 && (long long)(kDirectK + 1) * M * 4 <= 48 * 1024;
}

// The forward of gb_conv_igemm for the shapes gb_conv_direct_ok accepts (same arguments, no ktab).
GB_EXPORT int gb_conv_direct_small(int dtype, const void* x, const void* w, const int* idx, const void* bias,
                                   void* y, int Nimg, int C, int S, int L, int T, int M, void* stream) {
  if (dtype != DT_BF16 && dtype != DT_F16) {
    gbh::set_error("gb_conv_direct_small: bf16 or fp16 tensors");
    return gbh::E_BAD_ARG;
  }
  if (!gb_conv_direct_ok(C, T, M) || Nimg <= 0 || Nimg > 65535 || L <= 0) {
    gbh::set_error("gb_conv_direct_small: needs C * T <= %d, a channel count that is a multiple of 4, at most 65535 images", kDirectK);
    return gbh::E_BAD_ARG;
  }
  const size_t smem = (size_t)(kDirectK + 1) * M * sizeof(float);
  dim3 grid((L + 255) / 256, Nimg);
  conv_direct_small_kernel<kDirectK><<<grid, 256, smem, (cudaStream_t)stream>>>(
      (const uint16_t*)x, (const uint16_t*)w, idx, (const uint16_t*)bias, (uint16_t*)y, C, S, L, T, M, dtype == DT_BF16);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Number of K splits the weight gradient uses for a problem (partials: splits * M * C * T floats).
GB_EXPORT int gb_conv_wgrad_splits(int Nimg, int L, int M, int C, int T) {
  const long long R = (long long)Nimg * L;
  if (wgrad_small_ok(C, T, M)) return wgrad_small_ctas(R);      // one partial matrix per CTA of the direct kernel
  const long long tiles = (long long)((M + CBM - 1) / CBM) * ((C * T + CBN - 1) / CBN);
  long long want = (2 * 148 + tiles - 1) / tiles;          // about two waves of CTAs
  const long long max_splits = (R + 4 * CBK - 1) / (4 * CBK);  // at least four k-blocks per split
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  return (int)want;
}

// dW[m][(c,tap)] (+)= sum_{n,l} dy[n][m][l] * x[n][c][idx[l][tap]].  part: gb_conv_wgrad_splits() * M * C * T floats.
GB_EXPORT int gb_conv_wgrad(int dtype, const void* x, const void* dy, const int* ktab, const int* idx, void* dw,
                            float* part, int Nimg, int C, int S, int L, int T, int M, int beta, void* stream) {
  if (dtype != DT_BF16 && dtype != DT_F16) {
    gbh::set_error("gb_conv_wgrad: bf16 or fp16 tensors");
    return gbh::E_BAD_ARG;
  }
  if (T > CMAX_T_SMEM || (long long)C * S >= (1LL << 31) || (long long)M * L >= (1LL << 31)) {
    gbh::set_error("gb_conv_wgrad: geometry out of range");
    return gbh::E_BAD_ARG;
  }
  int rc = set_attr_once();
  if (rc) return rc;
  const int splits = gb_conv_wgrad_splits(Nimg, L, M, C, T);
  const long long R = (long long)Nimg * L;
  if (wgrad_small_ok(C, T, M)) {
    const size_t smem = (size_t)256 * ((kDirectK + 4) + (M + 4)) * sizeof(float);
    const int bf = dtype == DT_BF16;
#define GB_WS(MM)                                                                                              \
  {                                                                                                            \
    static bool cfg = false;                                                                                   \
    if (!cfg) {                                                                                                \
      GB_CUDA_OK(cudaFuncSetAttribute(conv_wgrad_small_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      cfg = true;                                                                                              \
    }                                                                                                          \
    conv_wgrad_small_kernel<MM><<<splits, 256, smem, (cudaStream_t)stream>>>(                                  \
        (const uint16_t*)x, (const uint16_t*)dy, idx, part, Nimg, C, S, L, T, bf);                             \
  }
    if (M == 32) GB_WS(32) else if (M == 64) GB_WS(64) else GB_WS(128)
#undef GB_WS
    const long long nn = (long long)M * C * T;
    conv_wgrad_finish_kernel<<<(int)((nn + 255) / 256 < 592 ? (nn + 255) / 256 : 592), 256, 0, (cudaStream_t)stream>>>(
        part, (uint16_t*)dw, nn, splits, bf, beta);
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  long long per = (R + splits - 1) / splits;
  per = (per + CBK - 1) / CBK * CBK;
  ConvArgs a;
  memset(&a, 0, sizeof(a));
  a.X = (const uint16_t*)x; a.DY = (const uint16_t*)dy; a.idx = idx; a.Y = part;
  a.ktab = (const int2*)ktab;
  a.Nimg = Nimg; a.C = C; a.S = S; a.L = L; a.T = T; a.M = M;
  a.bf16 = dtype == DT_BF16;
  a.r_per_split = per;
  a.status = gbh::status_ptr();
  const int K = C * T;
  dim3 grid((K + CBN - 1) / CBN, (M + CBM - 1) / CBM, splits);
  conv_igemm_kernel<1><<<grid, CTHREADS, CSMEM, (cudaStream_t)stream>>>(a);
  const long long n = (long long)M * K;
  conv_wgrad_finish_kernel<<<(int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592), 256, 0, (cudaStream_t)stream>>>(
      part, (uint16_t*)dw, n, splits, a.bf16, beta);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
