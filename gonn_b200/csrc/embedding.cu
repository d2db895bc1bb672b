// Embedding row gather (forward) and a deterministic scatter-add (backward).
//
// Backward builds, with a counting sort over the vocabulary, the list of token
// positions for every row, orders each list by position, and then one warp per
// vocabulary row sums its gradient rows in that order: no floating-point
// atomics, the result is independent of scheduling.  Rows nobody referenced are
// written as zeros, so the caller need not clear the output.
//
// The reference's Embedding is IndexSelect with a scatter-add backward on the
// host (tensor/ops_index.go:7-113, nn/embedding.go:108-126).
#include "bounds.cuh"

using namespace gb;

namespace {

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ w, const long long* __restrict__ idx,
                                   T* __restrict__ out, long long n, int D, long long V, int vec_ok,
                                   int* status) {
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long r = (long long)blockIdx.x * warps + warp; r < n; r += (long long)gridDim.x * warps) {
    long long v = idx[r];
    if (v < 0 || v >= V) {
      if (lane == 0) set_status(status, ST_BAD_INDEX, (int)r);
      v = 0;
    }
    const T* src = w + v * D;
    T* dst = out + r * D;
    if (vec_ok) {
      constexpr int VE = 16 / sizeof(T);
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int i = lane; i < D / VE; i += 32) d4[i] = s4[i];
    } else {
      for (int i = lane; i < D; i += 32) dst[i] = src[i];
    }
  }
}

__global__ void emb_count_kernel(const long long* __restrict__ idx, long long n, long long V,
                                 int* __restrict__ count) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    long long v = idx[i];
    if (v >= 0 && v < V) atomicAdd(&count[v], 1);
  }
}

// exclusive scan of count[0..V) into offs[0..V]; single CTA of 1024 threads.  Every thread owns a
// contiguous run of counters (whole cache lines once V >= 32 K), the 1024 run totals are scanned with
// warp shuffles (two levels), and the second pass re-reads the run from L1.
__global__ void emb_scan_kernel(const int* __restrict__ count, int V, int* __restrict__ offs) {
  __shared__ int warp_tot[32];
  const int per = (V + 1023) / 1024;
  const int b = threadIdx.x * per, e = min(b + per, V);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  // whole 16-byte groups when every thread's run is a multiple of four counters and starts aligned
  const bool vec = (per & 3) == 0 && e - b == per && ((uintptr_t)count & 15) == 0 && ((uintptr_t)offs & 15) == 0;
  int s = 0;
  if (vec) {
    const int4* c4 = reinterpret_cast<const int4*>(count + b);
#pragma unroll 8
    for (int i = 0; i < per / 4; i++) {
      const int4 v = c4[i];
      s += v.x + v.y + v.z + v.w;
    }
  } else {
#pragma unroll 8
    for (int i = b; i < e; i++) s += count[i];
  }
  int inc = s;                                           // inclusive scan inside the warp
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    const int w = warp_tot[lane];
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += t;
    }
    warp_tot[lane] = winc - w;                           // exclusive prefix of the warp totals
    if (lane == 31) offs[V] = winc;
  }
  __syncthreads();
  int run = warp_tot[wid] + inc - s;
  if (vec) {
    const int4* c4 = reinterpret_cast<const int4*>(count + b);
    int4* o4 = reinterpret_cast<int4*>(offs + b);
#pragma unroll 8
    for (int i = 0; i < per / 4; i++) {
      const int4 v = c4[i];
      int4 o;
      o.x = run; o.y = o.x + v.x; o.z = o.y + v.y; o.w = o.z + v.z;
      run = o.w + v.w;
      o4[i] = o;
    }
  } else {
#pragma unroll 8
    for (int i = b; i < e; i++) { offs[i] = run; run += count[i]; }
  }
}

__global__ void emb_place_kernel(const long long* __restrict__ idx, long long n, long long V,
                                 const int* __restrict__ offs, int* __restrict__ cursor,
                                 int* __restrict__ perm_tmp) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    long long v = idx[i];
    if (v >= 0 && v < V) {
      const int slot = offs[v] + atomicAdd(&cursor[v], 1);
      if (GB_IN_BOUNDS(slot, n, 201)) perm_tmp[slot] = (int)i;
    }
  }
}

// orders every segment by token position: rank = number of smaller positions
__global__ void emb_rank_kernel(const long long* __restrict__ idx, long long n, long long V,
                                const int* __restrict__ offs, const int* __restrict__ perm_tmp,
                                int* __restrict__ perm) {
  for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < n;
       s += (long long)gridDim.x * blockDim.x) {
    // slot s belongs to the vocabulary row of the token stored there
    const int pos = perm_tmp[s];
    if (pos < 0 || !GB_IN_BOUNDS(pos, n, 202)) continue;
    const long long v = idx[pos];
    if (!GB_IN_BOUNDS(v, V, 203)) continue;
    const int b = offs[v], e = offs[v + 1];
    if (!GB_IN_BOUNDS(e, n + 1, 204)) continue;
    int rank = 0;
    for (int j = b; j < e; j++) rank += perm_tmp[j] < pos;
    if (GB_IN_BOUNDS(b + rank, n, 205)) perm[b + rank] = pos;
  }
}

template <typename T> struct EAcc { using CT = float; };
template <> struct EAcc<double> { using CT = double; };

template <typename T, typename TO>
__global__ void emb_reduce_kernel(const T* __restrict__ dy, const int* __restrict__ offs,
                                  const int* __restrict__ perm, TO* __restrict__ dw, long long V,
                                  int D, long long padding_idx, int accumulate, long long n) {
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long v = (long long)blockIdx.x * warps + warp; v < V; v += (long long)gridDim.x * warps) {
    const int b = offs[v], e = (v == padding_idx) ? b : offs[v + 1];
    TO* out = dw + v * D;
    for (int c0 = lane * 4; c0 < D; c0 += 128) {
      using CT = typename EAcc<T>::CT;
      CT a0 = 0, a1 = 0, a2 = 0, a3 = 0;
      for (int j = b; j < e; j++) {
        if (!GB_IN_BOUNDS(j, n, 206) || !GB_IN_BOUNDS(perm[j], n, 207)) break;
        const T* src = dy + (long long)perm[j] * D + c0;
        a0 += (CT)src[0];
        if (c0 + 1 < D) a1 += (CT)src[1];
        if (c0 + 2 < D) a2 += (CT)src[2];
        if (c0 + 3 < D) a3 += (CT)src[3];
      }
      if (accumulate) {
        a0 += (CT)out[c0];
        if (c0 + 1 < D) a1 += (CT)out[c0 + 1];
        if (c0 + 2 < D) a2 += (CT)out[c0 + 2];
        if (c0 + 3 < D) a3 += (CT)out[c0 + 3];
      }
      out[c0] = (TO)a0;
      if (c0 + 1 < D) out[c0 + 1] = (TO)a1;
      if (c0 + 2 < D) out[c0 + 2] = (TO)a2;
      if (c0 + 3 < D) out[c0 + 3] = (TO)a3;
    }
  }
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// out[r, :] = w[idx[r], :]
GB_EXPORT int gb_gather_rows(int dtype, const void* w, const long long* idx, void* out, long long n,
                             int D, long long V, void* stream) {
  if (n <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = dtype == DT_F64 ? 8 : (dtype == DT_F32 ? 4 : 2);
  const int ve = 16 / esz;
  const int vec_ok = (D % ve == 0) && ((((uintptr_t)w | (uintptr_t)out) & 15) == 0);
  long long g = (n + 7) / 8;
  if (g > 148 * 8) g = 148 * 8;
  int* st = gbh::status_ptr();
  switch (dtype) {
    case DT_BF16: case DT_F16:
      gather_rows_kernel<uint16_t><<<(int)g, 256, 0, s>>>((const uint16_t*)w, idx, (uint16_t*)out, n, D, V, vec_ok, st);
      break;
    case DT_F32:
      gather_rows_kernel<float><<<(int)g, 256, 0, s>>>((const float*)w, idx, (float*)out, n, D, V, vec_ok, st);
      break;
    case DT_F64:
      gather_rows_kernel<double><<<(int)g, 256, 0, s>>>((const double*)w, idx, (double*)out, n, D, V, vec_ok, st);
      break;
    default:
      gbh::set_error("gb_gather_rows: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Number of ints of scratch the backward needs for n tokens and V rows.
GB_EXPORT long long gb_embedding_bwd_scratch_ints(long long n, long long V) {
  return 3 * V + 1 + 2 * n;
}

// dw[v, :] (+)= sum over tokens r with idx[r] == v of dy[r, :], rows summed in
// token order.  scratch: gb_embedding_bwd_scratch_ints(n, V) ints (contents
// arbitrary on entry).  out_dtype may be fp32 for bf16 / fp16 inputs.
GB_EXPORT int gb_embedding_bwd(int dtype, int out_dtype, const void* dy, const long long* idx,
                               void* dw, long long n, int D, long long V, long long padding_idx,
                               int accumulate, int* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (V <= 0 || D <= 0) return gbh::E_OK;
  GB_BOUNDS_BIND();
  if (n > 0x7fffffffLL || V > 0x7fffffffLL) {
    gbh::set_error("gb_embedding_bwd: sizes beyond 2^31 are not supported");
    return gbh::E_TOO_LARGE;
  }
  int* count = scratch;
  int* cursor = scratch + V;
  int* offs = scratch + 2 * V;       // V + 1 entries
  int* perm_tmp = offs + V + 1;
  int* perm = perm_tmp + n;
  GB_CUDA_OK(cudaMemsetAsync(count, 0, 2 * V * sizeof(int), s));
  if (n > 0) {
    GB_CUDA_OK(cudaMemsetAsync(perm_tmp, 0xff, n * sizeof(int), s));
    int g = (int)((n + 255) / 256);
    if (g > 148 * 8) g = 148 * 8;
    emb_count_kernel<<<g, 256, 0, s>>>(idx, n, V, count);
    emb_scan_kernel<<<1, 1024, 0, s>>>(count, (int)V, offs);
    emb_place_kernel<<<g, 256, 0, s>>>(idx, n, V, offs, cursor, perm_tmp);
    emb_rank_kernel<<<g, 256, 0, s>>>(idx, n, V, offs, perm_tmp, perm);
  } else {
    GB_CUDA_OK(cudaMemsetAsync(offs, 0, (V + 1) * sizeof(int), s));
  }
  long long g2 = (V + 7) / 8;
  if (g2 > 148 * 16) g2 = 148 * 16;
#define GB_E(T, TO) emb_reduce_kernel<T, TO><<<(int)g2, 256, 0, s>>>((const T*)dy, offs, perm, (TO*)dw, V, D, padding_idx, accumulate, n)
  if (dtype == DT_BF16 && out_dtype == DT_BF16) GB_E(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == DT_BF16 && out_dtype == DT_F32) GB_E(__nv_bfloat16, float);
  else if (dtype == DT_F16 && out_dtype == DT_F16) GB_E(__half, __half);
  else if (dtype == DT_F16 && out_dtype == DT_F32) GB_E(__half, float);
  else if (dtype == DT_F32 && out_dtype == DT_F32) GB_E(float, float);
  else if (dtype == DT_F64 && out_dtype == DT_F64) GB_E(double, double);
  else {
    gbh::set_error("gb_embedding_bwd: unsupported dtype pair %d -> %d", dtype, out_dtype);
    return gbh::E_BAD_ARG;
  }
#undef GB_E
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
