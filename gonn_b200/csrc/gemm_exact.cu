// Exact-precision GEMMs on tensor cores.
//
// The reference's float64 / float32 products are cuBLAS Dgemm / Sgemm calls
// (backend/cuda/gonn_cuda.cu:147-177, 255-294, 616-622).  tcgen05 has no fp64 or fp32 form, so:
//
// * fp64: a double-precision tensor-core main loop (mma.sync m8n8k4 f64): 128 x 128 x 16 CTA
//   tiles, sixteen warps of 32 x 32, operands staged through a three-deep cp.async ring in a
//   [k][m] layout whose padding makes every fragment load conflict-free.  Results match an
//   fp64 FMA chain in k order within a tile (1e-13-class agreement with a float64 oracle).
// * fp32: each operand is split once into three bf16 planes (x = hi + mid + lo, 24 mantissa
//   bits in total) and the six significant plane products hi*hi, hi*mid, mid*hi, hi*lo,
//   lo*hi, mid*mid run as bf16 tcgen05 GEMMs over an extended K axis (six times the length in
//   total, in three passes by magnitude class), with fp32 accumulation in tensor memory.  The
//   dropped products are below 2^-24 of the result, the rounding level of an fp32 product itself.  Non-finite inputs keep their value in the hi
//   plane and contribute zero to the others.
//
// The in-library benchmark loops at the end mirror the reference's (gonn_cuda.cu:255-294,
// 532-592, 673-690): operands allocated once, five untimed calls, `iters` calls between two
// events, milliseconds per call returned.
#include "common.cuh"

using namespace gb;

extern "C" int gb_gemm16(const void* A, const void* B, void* C, const void* bias, int bias_f32, void* aux, int M,
                         int N, int K, int batch, int transA, int transB, long long lda, long long ldb,
                         long long ldc, long long ldaux, long long sA, long long sB, long long sC, long long sAux,
                         int in_dtype, int out_dtype, int act, int aux_mode, int beta, float alpha, int force_bn,
                         void* workspace, long long workspace_bytes, void* stream);
extern "C" int gb_gemm_simt(const void* A, const void* B, void* C, int M, int N, int K, int batch, int transA,
                            int transB, long long lda, long long ldb, long long ldc, long long sA, long long sB,
                            long long sC, int dtype, double alpha, int beta, void* stream);
extern "C" int gb_binary(int op, int dtype, const void* a, const void* b, void* c, long long n, int rank,
                         const long long* shape, const long long* sa, const long long* sb, void* stream);
extern "C" int gb_flash_fwd(int dtype, const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                            int Sq, int Sk, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                            long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                            long long o_sb, long long o_ss, long long o_sh, float scale, int causal, void* stream);

namespace {

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// ---------------------------------------------------------------------------
// fp64: mma.sync m8n8k4
// ---------------------------------------------------------------------------
#ifndef GB_F64_BK
#define GB_F64_BK 16        // k extent of a stage (a multiple of 16)
#endif
#ifndef GB_F64_STAGES
#define GB_F64_STAGES 3
#endif
constexpr int DBM = 128, DBN = 128, DBK = GB_F64_BK, DSTAGES = GB_F64_STAGES;
static_assert(DBK % 16 == 0 && DSTAGES >= 2, "stage shape");
constexpr int DLD = DBM + 4;  // row pitch of a [k][m] stage in doubles: fragment loads hit 16 distinct bank pairs
constexpr int DTHREADS = 512;
constexpr int DSTAGE_DOUBLES = 2 * DBK * DLD;

__device__ __forceinline__ void cp_async8(void* dst, const void* src, bool pred) {
  const int n = pred ? 8 : 0;  // src-size 0: the destination is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}
// m16n8k8: A (16 x 8): a0 (g, t), a1 (g + 8, t), a2 (g, t + 4), a3 (g + 8, t + 4); B (8 x 8): b0 (t, g),
// b1 (t + 4, g); C (16 x 8): c0, c1 (g, 2t + {0, 1}), c2, c3 (g + 8, 2t + {0, 1}); g = lane / 4, t = lane % 4.
__device__ __forceinline__ void dmma16(double (&c)[4], const double (&a)[4], const double (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
      : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

// Copies one operand tile into a [k][mn] stage.  `k_contig`: the operand is stored with k as
// the contiguous dimension ((mn, k) row-major), so the copy transposes (8-byte pieces);
// otherwise rows of the stage are contiguous in memory (16-byte pieces when aligned).
__device__ __forceinline__ void load_tile(double* st, const double* src, long long ld, bool k_contig, int mn0,
                                          int k0, int MN, int K, bool vec_ok) {
  const int tid = threadIdx.x;
  if (k_contig) {
    // 128 rows x DBK k: thread -> (row = tid / 4, DBK / 4 consecutive k)
    const int r = tid >> 2, kq = (tid & 3) * (DBK / 4);
    const long long row = (long long)mn0 + r;
#pragma unroll
    for (int i = 0; i < DBK / 4; i++) {
      const int k = k0 + kq + i;
      const bool ok = row < MN && k < K;
      cp_async8(st + (kq + i) * DLD + r, ok ? src + row * ld + k : src, ok);
    }
  } else {
    // DBK k rows x 128 contiguous, 16 rows per pass: thread -> (k = tid / 32, four consecutive doubles)
    const int c = (tid & 31) * 4;
#pragma unroll
    for (int pass = 0; pass < DBK / 16; pass++) {
      const int kk = pass * 16 + (tid >> 5);
      const int k = k0 + kk;
      const double* g = src + (long long)k * ld + mn0 + c;
      double* d = st + kk * DLD + c;
      if (vec_ok && k < K && mn0 + c + 3 < MN) {
        cp_async16(d, g, true);
        cp_async16(d + 2, g + 2, true);
      } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const bool ok = k < K && mn0 + c + i < MN;
          cp_async8(d + i, ok ? g + i : src, ok);
        }
      }
    }
  }
}

template <int SHAPE>   // 0: m8n8k4 instructions, 1: m16n8k8
__global__ void __launch_bounds__(DTHREADS, 1)
gemm_f64_mma_kernel(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C, int M, int N,
                    int K, int transA, int transB, long long lda, long long ldb, long long ldc, long long sA,
                    long long sB, long long sC, double alpha, int beta) {
  extern __shared__ __align__(16) double dsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;  // 4 x 4 warps of 32 x 32
  const int m0 = blockIdx.y * DBM, n0 = blockIdx.x * DBN;
  A += (long long)blockIdx.z * sA;
  B += (long long)blockIdx.z * sB;
  C += (long long)blockIdx.z * sC;
  // A as stored: (M, K) row-major (k contiguous) unless transA, then (K, M)
  // B as stored: (K, N) row-major (n contiguous) unless transB, then (N, K) (k contiguous)
  const bool a_kc = transA == 0, b_kc = transB != 0;
  const bool a_vec = ((lda & 1) == 0) && (((uintptr_t)A & 15) == 0);
  const bool b_vec = ((ldb & 1) == 0) && (((uintptr_t)B & 15) == 0);
  const int nk = (K + DBK - 1) / DBK;

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) { acc[i][j][0] = 0.0; acc[i][j][1] = 0.0; }

  auto issue = [&](int kt) {
    if (kt < nk) {
      double* st = dsm + (kt % DSTAGES) * DSTAGE_DOUBLES;
      load_tile(st, A, lda, a_kc, m0, kt * DBK, M, K, a_vec);
      load_tile(st + DBK * DLD, B, ldb, b_kc, n0, kt * DBK, N, K, b_vec);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < DSTAGES - 1; i++) issue(i);
  const int fr = lane >> 2, fk = lane & 3;
  for (int kt = 0; kt < nk; kt++) {
    cp_async_wait<DSTAGES - 2>();   // tile kt has landed (the newer groups may still be in flight)
    __syncthreads();                // ... for every thread, and tile kt-1's stage is no longer read
    issue(kt + DSTAGES - 1);
    const double* sa = dsm + (kt % DSTAGES) * DSTAGE_DOUBLES;
    const double* sb = sa + DBK * DLD;
    if (SHAPE == 0) {
#pragma unroll
      for (int ks = 0; ks < DBK; ks += 4) {
        double af[4], bf[4];
#pragma unroll
        for (int i = 0; i < 4; i++) af[i] = sa[(ks + fk) * DLD + wm + i * 8 + fr];
#pragma unroll
        for (int j = 0; j < 4; j++) bf[j] = sb[(ks + fk) * DLD + wn + j * 8 + fr];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) dmma(acc[i][j][0], acc[i][j][1], af[i], bf[j]);
      }
    } else {
      // acc[2h][j] / acc[2h + 1][j] are the upper / lower 8 rows of 16-row tile h
#pragma unroll
      for (int ks = 0; ks < DBK; ks += 8) {
        double af[2][4], bf[4][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
          af[h][0] = sa[(ks + fk) * DLD + wm + h * 16 + fr];
          af[h][1] = sa[(ks + fk) * DLD + wm + h * 16 + 8 + fr];
          af[h][2] = sa[(ks + fk + 4) * DLD + wm + h * 16 + fr];
          af[h][3] = sa[(ks + fk + 4) * DLD + wm + h * 16 + 8 + fr];
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          bf[j][0] = sb[(ks + fk) * DLD + wn + j * 8 + fr];
          bf[j][1] = sb[(ks + fk + 4) * DLD + wn + j * 8 + fr];
        }
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            double c[4] = {acc[2 * h][j][0], acc[2 * h][j][1], acc[2 * h + 1][j][0], acc[2 * h + 1][j][1]};
            dmma16(c, af[h], bf[j]);
            acc[2 * h][j][0] = c[0]; acc[2 * h][j][1] = c[1];
            acc[2 * h + 1][j][0] = c[2]; acc[2 * h + 1][j][1] = c[3];
          }
      }
    }
  }
  cp_async_wait<0>();
  // C fragment: row = lane / 4, columns 2 * (lane % 4) + {0, 1} of each 8 x 8 tile
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + wm + i * 8 + fr;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + wn + j * 8 + 2 * fk;
      double* c = C + (long long)m * ldc + n;
      double v0 = alpha * acc[i][j][0], v1 = alpha * acc[i][j][1];
      if (n + 1 < N) {
        if (beta) { v0 += c[0]; v1 += c[1]; }
        c[0] = v0; c[1] = v1;
      } else if (n < N) {
        if (beta) v0 += c[0];
        c[0] = v0;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// fp32 as three bf16 planes
// ---------------------------------------------------------------------------
// Plane order along the extended K axis: A side (hi, hi, mid, hi, lo, mid), B side
// (hi, mid, hi, lo, hi, mid): position p of one multiplies position p of the other.
__constant__ int c_plane_a[6] = {0, 0, 1, 0, 2, 1};
__constant__ int c_plane_b[6] = {0, 1, 0, 2, 0, 1};

// src: (rows, cols) fp32 with row pitch ld.  k_contig: cols is the K axis and the six planes sit
// side by side in a row of 6 * Kp (Kp = cols padded to a multiple of 8, zero filled);
// otherwise rows is the K axis and the planes are stacked: plane p occupies rows [p * rows, (p+1) * rows).
__global__ void split3_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                              long long cols, long long ld, long long cols_p, int k_contig, int b_side,
                              long long src_batch, long long dst_batch) {
  src += (long long)blockIdx.z * src_batch;
  dst += (long long)blockIdx.z * dst_batch;
  const long long total = rows * cols_p;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols_p, c = i - r * cols_p;
    float x = c < cols ? src[r * ld + c] : 0.f;
    __nv_bfloat16 pl[3];
    if (isfinite(x)) {
      pl[0] = __float2bfloat16_rn(x);
      const float r1 = x - __bfloat162float(pl[0]);
      pl[1] = __float2bfloat16_rn(r1);
      pl[2] = __float2bfloat16_rn(r1 - __bfloat162float(pl[1]));
    } else {
      pl[0] = __float2bfloat16_rn(x);
      pl[1] = pl[2] = __float2bfloat16_rn(0.f);
    }
#pragma unroll
    for (int p = 0; p < 6; p++) {
      const __nv_bfloat16 v = pl[b_side ? c_plane_b[p] : c_plane_a[p]];
      if (k_contig) dst[r * (6 * cols_p) + p * cols_p + c] = v;
      else dst[((long long)p * rows + r) * cols_p + c] = v;
    }
  }
}

}  // namespace

namespace { int g_f64_shape = 1; }
// Instruction shape of the fp64 kernel: 0 = m8n8k4, 1 = m16n8k8 (default).
GB_EXPORT int gb_gemm_f64_tune(int shape) {
  g_f64_shape = shape ? 1 : 0;
  return gbh::E_OK;
}

// C = alpha * op(A) op(B) (+ C) in float64 on the double-precision tensor cores.
GB_EXPORT int gb_gemm_f64(const void* A, const void* B, void* C, int M, int N, int K, int batch, int transA,
                          int transB, long long lda, long long ldb, long long ldc, long long sA, long long sB,
                          long long sC, double alpha, int beta, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) {
    gbh::set_error("gb_gemm_f64: empty problem");
    return gbh::E_BAD_ARG;
  }
  dim3 grid((N + DBN - 1) / DBN, (M + DBM - 1) / DBM, batch);
  if (grid.y > 65535 || grid.z > 65535) {
    gbh::set_error("gb_gemm_f64: problem too large");
    return gbh::E_TOO_LARGE;
  }
  const size_t smem = (size_t)DSTAGES * DSTAGE_DOUBLES * sizeof(double);
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA_OK(cudaFuncSetAttribute(gemm_f64_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    GB_CUDA_OK(cudaFuncSetAttribute(gemm_f64_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set = true;
  }
  if (g_f64_shape == 0)
    gemm_f64_mma_kernel<0><<<grid, DTHREADS, smem, (cudaStream_t)stream>>>(
        (const double*)A, (const double*)B, (double*)C, M, N, K, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta);
  else
    gemm_f64_mma_kernel<1><<<grid, DTHREADS, smem, (cudaStream_t)stream>>>(
        (const double*)A, (const double*)B, (double*)C, M, N, K, transA, transB, lda, ldb, ldc, sA, sB, sC, alpha, beta);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Bytes of scratch gb_gemm_f32x3 needs for the split operands.
GB_EXPORT long long gb_gemm_f32x3_workspace(int M, int N, int K, int batch) {
  const long long Kp = (K + 7) / 8 * 8, Mp = (M + 7) / 8 * 8, Np = (N + 7) / 8 * 8;
  // either layout of an operand fits in 6 * Kp * (padded other dimension) elements
  return 2LL * batch * 6 * Kp * (Mp > Np ? Mp : Np) * 2 + 256;
}

// fp32 GEMM through three bf16 planes per operand (see the file header).  workspace:
// gb_gemm_f32x3_workspace() bytes; split_ws / split_ws_bytes: optional split-K scratch handed
// on to the bf16 GEMM.
GB_EXPORT int gb_gemm_f32x3(const void* A, const void* B, void* C, int M, int N, int K, int batch, int transA,
                            int transB, long long lda, long long ldb, long long ldc, long long sA, long long sB,
                            long long sC, float alpha, int beta, void* workspace, long long workspace_bytes,
                            void* split_ws, long long split_ws_bytes, void* stream) {
  if (workspace == nullptr || workspace_bytes < gb_gemm_f32x3_workspace(M, N, K, batch)) {
    gbh::set_error("gb_gemm_f32x3: workspace too small");
    return gbh::E_BAD_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const long long Kp = (K + 7) / 8 * 8, Mp = (M + 7) / 8 * 8, Np = (N + 7) / 8 * 8;
  __nv_bfloat16* a3 = (__nv_bfloat16*)workspace;
  const long long a_elems = 6 * Kp * Mp, b_elems = 6 * Kp * Np;
  __nv_bfloat16* b3 = a3 + (long long)batch * a_elems;
  const int ba = sA ? batch : 1, bb = sB ? batch : 1;
  long long lda3, ldb3;
  // A as stored: (M, K) (k contiguous) unless transA, then (K, M)
  if (!transA) {
    split3_kernel<<<dim3(592, 1, ba), 256, 0, s>>>((const float*)A, a3, M, K, lda, Kp, 1, 0, sA, a_elems);
    lda3 = 6 * Kp;
  } else {
    split3_kernel<<<dim3(592, 1, ba), 256, 0, s>>>((const float*)A, a3, K, M, lda, Mp, 0, 0, sA, a_elems);
    lda3 = Mp;
  }
  if (transB) {  // stored (N, K): k contiguous
    split3_kernel<<<dim3(592, 1, bb), 256, 0, s>>>((const float*)B, b3, N, K, ldb, Kp, 1, 1, sB, b_elems);
    ldb3 = 6 * Kp;
  } else {
    split3_kernel<<<dim3(592, 1, bb), 256, 0, s>>>((const float*)B, b3, K, N, ldb, Np, 0, 1, sB, b_elems);
    ldb3 = Np;
  }
  GB_CUDA_OK(cudaGetLastError());
  // Both operands must agree on where plane p starts along the extended K axis: at p * Kp when
  // the planes sit side by side, at p * K when they are stacked; so the stacked form needs Kp == K.
  const bool stacked_a = transA != 0, stacked_b = transB == 0;
  if ((stacked_a || stacked_b) && Kp != K) {
    gbh::set_error("gb_gemm_f32x3: K must be a multiple of 8 unless both operands are K-contiguous");
    return gbh::E_BAD_ARG;
  }
  // Three passes over sub-ranges of the extended K axis, smallest terms first, each added to C
  // by the epilogue's fp32 add: (hi*lo, lo*hi, mid*mid), then (hi*mid, mid*hi), then hi*hi.  The
  // tensor core aligns every product with its accumulator before adding; keeping terms of one
  // magnitude class per accumulator is what preserves the low planes' contribution.
  const int first_plane[3] = {3, 1, 0}, planes[3] = {3, 2, 1};
  for (int pass = 0; pass < 3; pass++) {
    const long long koff = (long long)first_plane[pass] * Kp;
    const __nv_bfloat16* ap = a3 + (stacked_a ? koff * lda3 : koff);
    const __nv_bfloat16* bp = b3 + (stacked_b ? koff * ldb3 : koff);
    const int rc = gb_gemm16(ap, bp, C, nullptr, 0, nullptr, M, N, (int)(planes[pass] * Kp), batch, transA, transB,
                             lda3, ldb3, ldc, 0, sA ? a_elems : 0, sB ? b_elems : 0, sC, 0, DT_BF16, DT_F32, 0, 0,
                             pass == 0 ? beta : 1, alpha, 0, split_ws, split_ws_bytes, stream);
    if (rc != 0) return rc;
  }
  return gbh::E_OK;
}

// ---------------------------------------------------------------------------
// in-library benchmark loops (milliseconds per call; -1 on an allocation failure)
// ---------------------------------------------------------------------------
namespace {
template <typename F>
double bench_loop(int iters, F&& fn) {
  for (int i = 0; i < 5; i++)
    if (fn() != 0) return -2.0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2.0;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int i = 0; i < iters; i++) fn();
  cudaEventRecord(e1);
  cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return (double)ms / iters;
}
}  // namespace

// Resident (m,k) @ (k,n).  dtype: 0 bf16, 1 fp16 (tcgen05, fp32 accumulate, operand bytes zeroed
// like the reference's fp16 loop), 2 fp32 (three-plane path), 3 fp64 (tensor-core fp64); the
// fp32 / fp64 operand bytes are set to 0x01 like the reference's loop.
GB_EXPORT double gb_bench_matmul(int m, int k, int n, int iters, int dtype) {
  const size_t esz = dtype == DT_F64 ? 8 : (dtype == DT_F32 ? 4 : 2);
  void *A = nullptr, *B = nullptr, *C = nullptr, *ws = nullptr;
  if (cudaMalloc(&A, esz * (size_t)m * k) != cudaSuccess) return -1.0;
  if (cudaMalloc(&B, esz * (size_t)k * n) != cudaSuccess) { cudaFree(A); return -1.0; }
  if (cudaMalloc(&C, esz * (size_t)m * n) != cudaSuccess) { cudaFree(A); cudaFree(B); return -1.0; }
  const int fill = esz == 2 ? 0 : 1;
  cudaMemset(A, fill, esz * (size_t)m * k);
  cudaMemset(B, fill, esz * (size_t)k * n);
  long long ws_bytes = 0;
  if (dtype == DT_F32) {
    ws_bytes = gb_gemm_f32x3_workspace(m, n, k, 1);
    if (cudaMalloc(&ws, ws_bytes) != cudaSuccess) { cudaFree(A); cudaFree(B); cudaFree(C); return -1.0; }
  }
  double ms;
  if (dtype == DT_F64)
    ms = bench_loop(iters, [&] { return gb_gemm_f64(A, B, C, m, n, k, 1, 0, 0, k, n, n, 0, 0, 0, 1.0, 0, nullptr); });
  else if (dtype == DT_F32)
    ms = bench_loop(iters, [&] {
      return gb_gemm_f32x3(A, B, C, m, n, k, 1, 0, 0, k, n, n, 0, 0, 0, 1.f, 0, ws, ws_bytes, nullptr, 0, nullptr);
    });
  else
    ms = bench_loop(iters, [&] {
      return gb_gemm16(A, B, C, nullptr, 0, nullptr, m, n, k, 1, 0, 0, k, n, n, 0, 0, 0, 0, 0, dtype, dtype, 0, 0, 0,
                       1.f, 0, nullptr, 0, nullptr);
    });
  cudaFree(A); cudaFree(B); cudaFree(C);
  if (ws) cudaFree(ws);
  return ms;
}

// Resident elementwise add of n elements (f32 != 0: float, else double).
GB_EXPORT double gb_bench_add(long long n, int iters, int f32) {
  const size_t esz = f32 ? 4 : 8;
  void *A = nullptr, *B = nullptr, *C = nullptr;
  if (cudaMalloc(&A, esz * n) != cudaSuccess) return -1.0;
  if (cudaMalloc(&B, esz * n) != cudaSuccess) { cudaFree(A); return -1.0; }
  if (cudaMalloc(&C, esz * n) != cudaSuccess) { cudaFree(A); cudaFree(B); return -1.0; }
  cudaMemset(A, 1, esz * n);
  cudaMemset(B, 1, esz * n);
  const double ms = bench_loop(iters, [&] { return gb_binary(0, f32 ? DT_F32 : DT_F64, A, B, C, n, 0, nullptr, nullptr, nullptr, nullptr); });
  cudaFree(A); cudaFree(B); cudaFree(C);
  return ms;
}

// Resident attention forward over (BH, S, d) in bf16 (d = 64 or 128), zero-filled like the reference's loop.
GB_EXPORT double gb_bench_flash_attn(int BH, int S, int d, int iters, int causal) {
  const size_t n = (size_t)BH * S * d;
  void *Q = nullptr, *K = nullptr, *V = nullptr, *O = nullptr;
  float* L = nullptr;
  if (cudaMalloc(&Q, 2 * n) != cudaSuccess) return -1.0;
  if (cudaMalloc(&K, 2 * n) != cudaSuccess) { cudaFree(Q); return -1.0; }
  if (cudaMalloc(&V, 2 * n) != cudaSuccess) { cudaFree(Q); cudaFree(K); return -1.0; }
  if (cudaMalloc(&O, 2 * n) != cudaSuccess) { cudaFree(Q); cudaFree(K); cudaFree(V); return -1.0; }
  if (cudaMalloc(&L, 4 * (size_t)BH * S) != cudaSuccess) { cudaFree(Q); cudaFree(K); cudaFree(V); cudaFree(O); return -1.0; }
  cudaMemset(Q, 0, 2 * n);
  cudaMemset(K, 0, 2 * n);
  cudaMemset(V, 0, 2 * n);
  // (BH, S, d) read as batch 1, BH heads: head stride S * d, sequence stride d
  const long long sb = (long long)n, ss = d, sh = (long long)S * d;
  const float scale = 1.f / sqrtf((float)d);
  const double ms = bench_loop(iters, [&] {
    return gb_flash_fwd(DT_BF16, Q, K, V, O, L, 1, BH, S, S, d, sb, ss, sh, sb, ss, sh, sb, ss, sh, sb, ss, sh, scale,
                        causal, nullptr);
  });
  cudaFree(Q); cudaFree(K); cudaFree(V); cudaFree(O); cudaFree(L);
  return ms;
}
