// General fused attention: additive / boolean masks, key-padding masks, attention dropout, any
// head size up to 128, bf16 / fp16 / fp32 / fp64.  No (Tq, Tk) score matrix is ever stored.
//
// This is the path of MultiHeadAttention.ForwardMasked (nn/attention.go:199-341: an additive
// -1e30 mask for masked pairs, the key-padding mask broadcast over heads and queries, dropout
// on the probabilities) and of attention in fp32 / fp64 (the reference's fused CUDA kernels are
// float64: backend/cuda/gonn_cuda.cu:302-450).  The unmasked 16-bit case runs on the tcgen05
// kernels of flash_attn.cu instead.
//
// One kernel body serves three roles.  A CTA of four warps owns 16 "rows" (four per warp) and
// streams the other side of the attention matrix in tiles of 32, one tile row per lane:
//   FWD   rows = queries, tiles = keys:   s = q.k  ->  online softmax  ->  o += p v
//   DQ    rows = queries, tiles = keys:   p = exp(s - lse), dp = dO.v, ds = p (dp' - delta) scale,
//                                          dq += ds k
//   DKV   rows = keys, tiles = queries:   the same p and ds (transposed roles), dv += p' dO, dk += ds q
// (p' / dp' = the dropout mask and 1/(1-p_drop) applied).  Every output element has one owner
// and a fixed summation order: bit-reproducible, no atomics (the reference's backward uses fp64
// atomicAdd).  The dropout mask comes from Philox-4x32-10 keyed by (seed, b, h, q / 4, k), one output word
// per query, so forward and both backward kernels regenerate it.
#include "common.cuh"

using namespace gb;

namespace {

constexpr int GR = 4;           // rows per warp
constexpr int GW = 4;           // warps per CTA
constexpr int GROWS = GR * GW;  // rows per CTA
constexpr int GT = 32;          // tile rows (one per lane)
static_assert(GR == 4, "the coefficient buffers are read four rows at a time; one dropout draw covers a warp's four rows");

enum { MODE_FWD = 0, MODE_DQ = 1, MODE_DKV = 2 };

struct GArgs {
  const void *Q, *K, *V, *dO;
  void *O, *dQ, *dK, *dV;
  void* LSE;             // [B, H, Tq], natural log; in the compute type (fp32, or fp64 for fp64 tensors)
  void* Delta;           // [B, H, Tq], same type
  long long q_s[3], k_s[3], v_s[3], o_s[3], g_s[3], dq_s[3], dk_s[3], dv_s[3];  // (b, s, h) element strides
  int B, H, Tq, Tk, D;
  double scale;
  int causal;
  const float* mask;            // [Tq, Tk] additive, or null
  const unsigned char* kpm;     // [B, Tk], 1 = padded key, or null
  double p_drop;
  unsigned long long seed;
};

__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; r++) {
    uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
// One Philox call serves the four queries 4g .. 4g+3 against key k: counter (g, k, bh), query q takes
// word q % 4.  A warp's four query rows (forward, dQ) start at a multiple of four, so there one call
// per lane and tile covers all four rows; the dK/dV role (rows are keys) draws once per cell.
__device__ __forceinline__ uint4 keep_draw(const GArgs& a, int bh, int qgroup, int k) {
  return philox(make_uint4((uint32_t)qgroup, (uint32_t)k, (uint32_t)bh, 0u),
                make_uint2((uint32_t)a.seed, (uint32_t)(a.seed >> 32)));
}
__device__ __forceinline__ uint32_t draw_word(const uint4& r, int i) {
  return i == 0 ? r.x : i == 1 ? r.y : i == 2 ? r.z : r.w;
}
__device__ __forceinline__ bool keep_cell(const GArgs& a, int bh, int q, int k, uint32_t thresh) {
  return draw_word(keep_draw(a, bh, q >> 2, k), q & 3) >= thresh;
}

template <typename T> struct Cvt {
  static __device__ __forceinline__ float ld(const T* p) { return (float)*p; }
};
template <typename T, typename CT> __device__ __forceinline__ CT load_as(const T* p) { return (CT)(*p); }
template <> __device__ __forceinline__ float load_as<__nv_bfloat16, float>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float load_as<__half, float>(const __half* p) { return __half2float(*p); }
template <typename T, typename CT> __device__ __forceinline__ T store_as(CT v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 store_as<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half store_as<__half, float>(float v) { return __float2half_rn(v); }

template <typename CT> __device__ __forceinline__ CT wsum(CT v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename CT> __device__ __forceinline__ CT wmax(CT v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { CT u = __shfl_xor_sync(0xffffffffu, v, o); v = u > v ? u : v; }
  return v;
}
__device__ __forceinline__ float exp_ct(float x) { return __expf(x); }
__device__ __forceinline__ double exp_ct(double x) { return exp(x); }
__device__ __forceinline__ float log_ct(float x) { return __logf(x); }
__device__ __forceinline__ double log_ct(double x) { return log(x); }

// Four consecutive elements of the compute type, read from / written to shared memory with 16-byte
// accesses (p is a multiple of four elements away from the 16-byte aligned base).
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld4(const double* p, double (&v)[4]) {
  const double2 t = *reinterpret_cast<const double2*>(p), u = *reinterpret_cast<const double2*>(p + 2);
  v[0] = t.x; v[1] = t.y; v[2] = u.x; v[3] = u.y;
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(double* p, const double (&v)[4]) {
  *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
  *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

// Four consecutive elements from global memory: one or two vector loads when `vec` (the address is
// aligned to min(16, 4 * sizeof(T)) bytes), else element by element.
template <typename T, typename CT>
__device__ __forceinline__ void gload4(const T* g, bool vec, CT (&v)[4]) {
  if (vec) {
    if constexpr (sizeof(T) == 8) {
      const double2 t = __ldg(reinterpret_cast<const double2*>(g)), u = __ldg(reinterpret_cast<const double2*>(g) + 1);
      v[0] = (CT)t.x; v[1] = (CT)t.y; v[2] = (CT)u.x; v[3] = (CT)u.y;
    } else if constexpr (sizeof(T) == 4) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(g));
      v[0] = (CT)t.x; v[1] = (CT)t.y; v[2] = (CT)t.z; v[3] = (CT)t.w;
    } else {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(g));
      T t[4];
      memcpy(t, &raw, 8);
#pragma unroll
      for (int u = 0; u < 4; u++) v[u] = load_as<T, CT>(t + u);
    }
  } else {
#pragma unroll
    for (int u = 0; u < 4; u++) v[u] = load_as<T, CT>(g + u);
  }
}

// Copies `n` rows of D elements (rows r0.. of tensor p with strides s, fixed b and h) into smem
// [n][DP]; rows past `limit` and the columns D .. round-up-to-4(D) become zero (nothing reads further).
// Head sizes that are multiples of 4 move in chunks of four elements, four chunks per thread in
// flight before the first is stored: the loop is bound by the L2 round trip otherwise.
template <typename T, typename CT>
__device__ __forceinline__ void stage_rows(CT* dst, const void* p, const long long* s, int b, int h, int r0, int n,
                                           int limit, int D, int DP) {
  const T* base = (const T*)p + (long long)b * s[0] + (long long)h * s[2];
  if ((D & 3) == 0) {
    constexpr int U = 4;
    constexpr uintptr_t AL = sizeof(T) * 4 < 16 ? sizeof(T) * 4 : 16;
    const bool vec = ((reinterpret_cast<uintptr_t>(base) | (uintptr_t)(s[1] * (long long)sizeof(T))) & (AL - 1)) == 0;
    const int nc = D >> 2, total = n * nc;
    for (int q0 = threadIdx.x; q0 < total; q0 += blockDim.x * U) {
      CT v[U][4];
      int off[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int q = q0 + u * blockDim.x;
#pragma unroll
        for (int c = 0; c < 4; c++) v[u][c] = 0;
        off[u] = -1;
        if (q < total) {
          const int r = q / nc, c = (q - r * nc) * 4;
          off[u] = r * DP + c;
          if (r0 + r < limit) gload4<T, CT>(base + (long long)(r0 + r) * s[1] + c, vec, v[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++)
        if (off[u] >= 0) st4(dst + off[u], v[u]);
    }
    return;
  }
  const int DR = (D + 3) & ~3;
  for (int i = threadIdx.x; i < n * DR; i += blockDim.x) {
    const int r = i / DR, c = i - r * DR;
    CT v = 0;
    if (c < D && r0 + r < limit) v = load_as<T, CT>(base + (long long)(r0 + r) * s[1] + c);
    dst[r * DP + c] = v;
  }
}

template <typename T, typename CT, int MODE>
__global__ void __launch_bounds__(GW * 32)
attn_general_kernel(const GArgs a) {
  extern __shared__ __align__(16) unsigned char gsm[];
  const int D = a.D;
  const int DP = (D + 3) / 4 * 4 + 4;        // row pitch: a multiple of 4 plus 4 (conflict-free float4 reads per lane)
  CT* rowsA = reinterpret_cast<CT*>(gsm);    // [GROWS][DP]  FWD/DQ: Q rows; DKV: K rows
  CT* rowsB = rowsA + GROWS * DP;            // [GROWS][DP]  DQ: dO rows; DKV: V rows (absent in FWD)
  CT* tileA = rowsB + (MODE == MODE_FWD ? 0 : GROWS * DP);   // [GT][DP]  FWD/DQ: K tile; DKV: Q tile
  CT* tileB = tileA + GT * DP;               // [GT][DP]     FWD/DQ: V tile; DKV: dO tile
  CT* pbuf = tileB + GT * DP;                // [GW][GT][GR] coefficients of the first accumulation
  CT* dbuf = pbuf + GW * GT * GR;            // [GW][GT][GR] coefficients of the second (DKV)
  CT* tstat = dbuf + GW * GT * GR;           // [2][GT] lse / delta of the tile's queries (DKV)
  CT* LSEp = reinterpret_cast<CT*>(a.LSE);
  const CT* Deltap = reinterpret_cast<const CT*>(a.Delta);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, bh = b * a.H + h;
  const int row0 = blockIdx.x * GROWS;                 // first row of the CTA
  const int nrows = MODE == MODE_DKV ? a.Tk : a.Tq;    // extent of the row side
  const int ntile = MODE == MODE_DKV ? a.Tq : a.Tk;    // extent of the streamed side
  const uint32_t thresh = (uint32_t)fmin(a.p_drop * 4294967296.0, 4294967295.0);
  const CT keep_scale = a.p_drop > 0.0 ? (CT)(1.0 / (1.0 - a.p_drop)) : (CT)1;
  const CT scale = (CT)a.scale;
  const CT NEG = (CT)-1e30;

  if (MODE == MODE_DKV) {
    stage_rows<T, CT>(rowsA, a.K, a.k_s, b, h, row0, GROWS, a.Tk, D, DP);
    stage_rows<T, CT>(rowsB, a.V, a.v_s, b, h, row0, GROWS, a.Tk, D, DP);
  } else {
    stage_rows<T, CT>(rowsA, a.Q, a.q_s, b, h, row0, GROWS, a.Tq, D, DP);
    if (MODE == MODE_DQ) stage_rows<T, CT>(rowsB, a.dO, a.g_s, b, h, row0, GROWS, a.Tq, D, DP);
  }

  // accumulators: lane owns columns 4*lane .. 4*lane+3 (d <= 128)
  CT acc[GR][4], acc2[GR][4];
  CT m[GR], l[GR], lse_r[GR], delta_r[GR];
#pragma unroll
  for (int r = 0; r < GR; r++) {
    m[r] = (CT)-INFINITY;
    l[r] = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) { acc[r][c] = 0; acc2[r][c] = 0; }
    const int row = row0 + warp * GR + r;
    lse_r[r] = 0;
    delta_r[r] = 0;
    if (MODE == MODE_DQ && row < a.Tq) {
      lse_r[r] = LSEp[(long long)bh * a.Tq + row];
      delta_r[r] = Deltap[(long long)bh * a.Tq + row];
    }
  }
  const int wrow0 = warp * GR;               // this warp's first row inside the CTA
  // A row of D columns needs ceil(D / 4) lanes in the accumulation step.  With head size <= 64 the
  // warp splits into 2 (or 4, head size <= 32) lane groups that take interleaved tile rows, so no
  // lane idles; the groups' partial sums meet after the last tile.
  const int nl = (D + 3) >> 2;
  const int groups = nl <= 8 ? 4 : nl <= 16 ? 2 : 1;
  const int lpg = 32 / groups;
  const int grp = lane / lpg, c0 = (lane - grp * lpg) * 4;
  // pure causal attention never looks past the diagonal: later tiles contribute exact zeros
  int tile_end = ntile;
  int tile_begin = 0;
  if (a.causal && a.mask == nullptr && a.kpm == nullptr) {
    if (MODE == MODE_DKV) tile_begin = row0 / GT * GT;                    // queries before the first key row see none of them
    else tile_end = min(ntile, row0 + GROWS);
  }

  for (int t0 = tile_begin; t0 < tile_end; t0 += GT) {
    __syncthreads();   // the previous tile is no longer read
    if (MODE == MODE_DKV) {
      stage_rows<T, CT>(tileA, a.Q, a.q_s, b, h, t0, GT, a.Tq, D, DP);
      stage_rows<T, CT>(tileB, a.dO, a.g_s, b, h, t0, GT, a.Tq, D, DP);
      if (threadIdx.x < GT) {
        const int qi = t0 + threadIdx.x;
        tstat[threadIdx.x] = qi < a.Tq ? LSEp[(long long)bh * a.Tq + qi] : (CT)0;
        tstat[GT + threadIdx.x] = qi < a.Tq ? Deltap[(long long)bh * a.Tq + qi] : (CT)0;
      }
    } else {
      stage_rows<T, CT>(tileA, a.K, a.k_s, b, h, t0, GT, a.Tk, D, DP);
      stage_rows<T, CT>(tileB, a.V, a.v_s, b, h, t0, GT, a.Tk, D, DP);
    }
    __syncthreads();

    const int tj = t0 + lane;                 // this lane's tile row (a key, or a query in DKV)
    const bool tvalid = tj < ntile;
    // ---- scores of the 4 rows against this lane's tile row (and dO.v products) ----
    CT s[GR], dp[GR];
#pragma unroll
    for (int r = 0; r < GR; r++) { s[r] = 0; dp[r] = 0; }
    {
      const CT* ta = tileA + lane * DP;
      const CT* tb = tileB + lane * DP;
      for (int c = 0; c < D; c += 4) {
        CT x[4], y[4];
        ld4(ta + c, x);
        if (MODE != MODE_FWD) ld4(tb + c, y);
#pragma unroll
        for (int r = 0; r < GR; r++) {
          CT q4[4];
          ld4(rowsA + (wrow0 + r) * DP + c, q4);
#pragma unroll
          for (int u = 0; u < 4; u++) s[r] += q4[u] * x[u];
          if (MODE != MODE_FWD) {
            CT g4[4];
            ld4(rowsB + (wrow0 + r) * DP + c, g4);
#pragma unroll
            for (int u = 0; u < 4; u++) dp[r] += g4[u] * y[u];
          }
        }
      }
    }
    // ---- masks, softmax terms ----
    CT coef[GR], coef2[GR];
    uint4 draw = make_uint4(0u, 0u, 0u, 0u);
    if (MODE != MODE_DKV && a.p_drop > 0.0 && tvalid) draw = keep_draw(a, bh, (row0 + wrow0) >> 2, tj);
#pragma unroll
    for (int r = 0; r < GR; r++) {
      const int row = row0 + wrow0 + r;
      const int qi = MODE == MODE_DKV ? tj : row, ki = MODE == MODE_DKV ? row : tj;
      const bool rvalid = row < nrows;
      CT sv = s[r] * scale;
      if (tvalid && rvalid) {
        if (a.causal && ki > qi) sv += NEG;
        if (a.mask) sv += (CT)a.mask[(long long)qi * a.Tk + ki];
        if (a.kpm && a.kpm[(long long)b * a.Tk + ki]) sv += NEG;
      }
      bool keep = true;
      if (a.p_drop > 0.0 && tvalid && rvalid)
        keep = MODE == MODE_DKV ? keep_cell(a, bh, qi, ki, thresh) : draw_word(draw, r) >= thresh;
      if (MODE == MODE_FWD) {
        // online softmax over the 32 lanes; tile rows past the end do not take part
        const CT sm = tvalid ? sv : (CT)-INFINITY;
        const CT m_new = fmax(m[r], wmax(sm));
        const CT p = tvalid ? exp_ct(sv - m_new) : (CT)0;
        if (m_new != m[r]) {      // warp-uniform; after the first tiles the running maximum rarely moves
          const CT corr = m[r] == (CT)-INFINITY ? (CT)0 : exp_ct(m[r] - m_new);
          l[r] *= corr;
#pragma unroll
          for (int c = 0; c < 4; c++) acc[r][c] *= corr;
          m[r] = m_new;
        }
        l[r] += wsum(p);
        coef[r] = keep ? p * keep_scale : (CT)0;
        coef2[r] = 0;
      } else {
        const CT lse = MODE == MODE_DKV ? tstat[lane] : lse_r[r];
        const CT delta = MODE == MODE_DKV ? tstat[GT + lane] : delta_r[r];
        const CT p = (tvalid && rvalid) ? exp_ct(sv - lse) : (CT)0;
        const CT dpd = keep ? dp[r] * keep_scale : (CT)0;
        const CT ds = p * (dpd - delta) * scale;
        coef[r] = ds;                                  // DQ: dq += ds k      DKV: dk += ds q
        coef2[r] = keep ? p * keep_scale : (CT)0;      //                      DKV: dv += p' dO
      }
    }
    // ---- hand the coefficients to the whole warp, then accumulate with lanes along columns ----
    __syncwarp();
    CT* pw = pbuf + (warp * GT + lane) * GR;
    CT* dw = dbuf + (warp * GT + lane) * GR;
#pragma unroll
    for (int r = 0; r < GR; r++) { pw[r] = coef[r]; if (MODE == MODE_DKV) dw[r] = coef2[r]; }
    __syncwarp();
    if (c0 < D) {
      // FWD: acc += p V      DQ: acc += ds K      DKV: acc += ds Q, acc2 += p' dO
      const CT* src1 = MODE == MODE_FWD ? tileB : tileA;
      for (int j = grp; j < GT; j += groups) {
        CT pj[4], v1[4];
        ld4(pbuf + (warp * GT + j) * GR, pj);
        ld4(src1 + j * DP + c0, v1);
#pragma unroll
        for (int r = 0; r < GR; r++)
#pragma unroll
          for (int c = 0; c < 4; c++) acc[r][c] += pj[r] * v1[c];
        if (MODE == MODE_DKV) {
          CT dj[4], v2[4];
          ld4(dbuf + (warp * GT + j) * GR, dj);
          ld4(tileB + j * DP + c0, v2);
#pragma unroll
          for (int r = 0; r < GR; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc2[r][c] += dj[r] * v2[c];
        }
      }
    }
  }

  // the lane groups hold partial sums over interleaved tile rows: add them up (fixed order)
  for (int o = lpg; o < 32; o <<= 1) {
#pragma unroll
    for (int r = 0; r < GR; r++)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        acc[r][c] += __shfl_xor_sync(0xffffffffu, acc[r][c], o);
        if (MODE == MODE_DKV) acc2[r][c] += __shfl_xor_sync(0xffffffffu, acc2[r][c], o);
      }
  }

  // ---- outputs (the first lane group writes) ----
#pragma unroll
  for (int r = 0; r < GR; r++) {
    const int row = row0 + wrow0 + r;
    if (row >= nrows || grp != 0) continue;
    if (MODE == MODE_FWD) {
      const CT inv = l[r] > 0 ? (CT)1 / l[r] : (CT)0;
      T* o = (T*)a.O + (long long)b * a.o_s[0] + (long long)row * a.o_s[1] + (long long)h * a.o_s[2];
      for (int c = 0; c < 4; c++)
        if (c0 + c < D) o[c0 + c] = store_as<T, CT>(acc[r][c] * inv);
      if (lane == 0 && LSEp) LSEp[(long long)bh * a.Tq + row] = l[r] > 0 ? m[r] + log_ct(l[r]) : (CT)-INFINITY;
    } else if (MODE == MODE_DQ) {
      T* o = (T*)a.dQ + (long long)b * a.dq_s[0] + (long long)row * a.dq_s[1] + (long long)h * a.dq_s[2];
      for (int c = 0; c < 4; c++)
        if (c0 + c < D) o[c0 + c] = store_as<T, CT>(acc[r][c]);
    } else {
      T* ok = (T*)a.dK + (long long)b * a.dk_s[0] + (long long)row * a.dk_s[1] + (long long)h * a.dk_s[2];
      T* ov = (T*)a.dV + (long long)b * a.dv_s[0] + (long long)row * a.dv_s[1] + (long long)h * a.dv_s[2];
      for (int c = 0; c < 4; c++)
        if (c0 + c < D) {
          ok[c0 + c] = store_as<T, CT>(acc[r][c]);
          ov[c0 + c] = store_as<T, CT>(acc2[r][c]);
        }
    }
  }
}

// delta[b][h][q] = sum_t dO[q][t] * O[q][t]
template <typename T, typename CT>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ g, CT* __restrict__ delta,
                                  int B, int H, int S, int D, long long o0, long long o1, long long o2,
                                  long long g0, long long g1, long long g2) {
  const long long total = (long long)B * H * S;
  const int lane = threadIdx.x & 31;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 5) {
    const int q = (int)(w % S);
    const int hh = (int)((w / S) % H);
    const int bb = (int)(w / ((long long)S * H));
    const T* op = o + bb * o0 + q * o1 + hh * o2;
    const T* gp = g + bb * g0 + q * g1 + hh * g2;
    CT sacc = 0;
    for (int t = lane; t < D; t += 32) sacc += load_as<T, CT>(op + t) * load_as<T, CT>(gp + t);
    sacc = wsum(sacc);
    if (lane == 0) delta[((long long)bb * H + hh) * S + q] = sacc;
  }
}

// The dropout keep-mask the kernels regenerate, written out for tests and debugging.
__global__ void attn_keep_mask_kernel(unsigned char* out, int B, int H, int Tq, int Tk, double p_drop,
                                      unsigned long long seed) {
  GArgs a;
  a.seed = seed;
  const uint32_t thresh = (uint32_t)fmin(p_drop * 4294967296.0, 4294967295.0);
  const long long total = (long long)B * H * Tq * Tk;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % Tk), q = (int)((i / Tk) % Tq), bh = (int)(i / ((long long)Tk * Tq));
    out[i] = keep_cell(a, bh, q, k, thresh) ? 1 : 0;
  }
}

// Shared memory of one CTA: every role has its rows, two tiles and one coefficient buffer; the backward
// roles add the second row block, dK/dV the second coefficient buffer and the tile's lse / delta.
template <typename CT>
size_t general_smem(int D, int mode) {
  const int DP = (D + 3) / 4 * 4 + 4;
  size_t elems = (size_t)(GROWS + 2 * GT) * DP + (size_t)GW * GT * GR;
  if (mode != MODE_FWD) elems += (size_t)GROWS * DP;
  if (mode == MODE_DKV) elems += (size_t)GW * GT * GR + 2 * GT;
  return elems * sizeof(CT);
}

template <typename T, typename CT>
int launch_general(int mode, const GArgs& a, cudaStream_t s) {
  const size_t smem = general_smem<CT>(a.D, mode);
  static bool set[3] = {false, false, false};
  auto k0 = attn_general_kernel<T, CT, MODE_FWD>;
  auto k1 = attn_general_kernel<T, CT, MODE_DQ>;
  auto k2 = attn_general_kernel<T, CT, MODE_DKV>;
  if (!set[mode]) {
    const int lim = (int)general_smem<CT>(128, mode);
    if (mode == 0) GB_CUDA_OK(cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    if (mode == 1) GB_CUDA_OK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    if (mode == 2) GB_CUDA_OK(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    set[mode] = true;
  }
  const int rows = mode == MODE_DKV ? a.Tk : a.Tq;
  dim3 grid((rows + GROWS - 1) / GROWS, a.H, a.B);
  if (mode == 0) k0<<<grid, GW * 32, smem, s>>>(a);
  else if (mode == 1) k1<<<grid, GW * 32, smem, s>>>(a);
  else k2<<<grid, GW * 32, smem, s>>>(a);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// out[b][h][q][k] = 1 where the attention weight survives dropout with this seed and probability.
GB_EXPORT int gb_attn_keep_mask(unsigned char* out, int B, int H, int Tq, int Tk, double p_drop, long long seed,
                                void* stream) {
  attn_keep_mask_kernel<<<592, 256, 0, (cudaStream_t)stream>>>(out, B, H, Tq, Tk, p_drop, (unsigned long long)seed);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// mode 0: forward (writes O and LSE); 1: dQ; 2: dK and dV (modes 1 and 2 first need delta: mode 3 computes
// it from O and dO).  ptrs: Q, K, V, dO, O, dQ, dK, dV (unused ones null); strides: 8 triples (b, s, h) in the
// same order.  lse / delta: (B, H, Tq) in fp32 (fp64 for fp64 tensors).  mask: additive fp32 (Tq, Tk) or null; kpm: bytes (B, Tk), non-zero = padded key, or null.
GB_EXPORT int gb_attn_general(int mode, int dtype, void* const* ptrs, const long long* strides, void* lse,
                              void* delta, int B, int H, int Tq, int Tk, int D, double scale, int causal,
                              const float* mask, const unsigned char* kpm, double p_drop, long long seed,
                              void* stream) {
  if (D < 1 || D > 128 || B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || B > 65535 || H > 65535) {
    gbh::set_error("gb_attn_general: bad shape (head size 1..128)");
    return gbh::E_BAD_ARG;
  }
  if (p_drop < 0.0 || p_drop >= 1.0) {
    gbh::set_error("gb_attn_general: dropout probability must be in [0, 1)");
    return gbh::E_BAD_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  GArgs a;
  memset(&a, 0, sizeof(a));
  a.Q = ptrs[0]; a.K = ptrs[1]; a.V = ptrs[2]; a.dO = ptrs[3];
  a.O = ptrs[4]; a.dQ = ptrs[5]; a.dK = ptrs[6]; a.dV = ptrs[7];
  long long* dst[8] = {a.q_s, a.k_s, a.v_s, a.g_s, a.o_s, a.dq_s, a.dk_s, a.dv_s};
  for (int i = 0; i < 8; i++)
    for (int j = 0; j < 3; j++) dst[i][j] = strides[i * 3 + j];
  a.LSE = lse; a.Delta = delta;
  a.B = B; a.H = H; a.Tq = Tq; a.Tk = Tk; a.D = D;
  a.scale = scale; a.causal = causal; a.mask = mask; a.kpm = kpm; a.p_drop = p_drop;
  a.seed = (unsigned long long)seed;
  if (mode == 3) {
    const long long warps = (long long)B * H * Tq;
    const int grid = (int)((warps * 32 + 255) / 256 < 148 * 16 ? (warps * 32 + 255) / 256 : 148 * 16);
#define GB_DELTA(T, CT)                                                                                              \
    attn_delta_kernel<T, CT><<<grid, 256, 0, s>>>((const T*)a.O, (const T*)a.dO, (CT*)delta, B, H, Tq, D, a.o_s[0], a.o_s[1], \
                                                  a.o_s[2], a.g_s[0], a.g_s[1], a.g_s[2])
    switch (dtype) {
      case DT_BF16: GB_DELTA(__nv_bfloat16, float); break;
      case DT_F16: GB_DELTA(__half, float); break;
      case DT_F32: GB_DELTA(float, float); break;
      case DT_F64: GB_DELTA(double, double); break;
      default: gbh::set_error("gb_attn_general: bad dtype %d", dtype); return gbh::E_BAD_ARG;
    }
#undef GB_DELTA
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  if (mode < 0 || mode > 2) {
    gbh::set_error("gb_attn_general: bad mode %d", mode);
    return gbh::E_BAD_ARG;
  }
  switch (dtype) {
    case DT_BF16: return launch_general<__nv_bfloat16, float>(mode, a, s);
    case DT_F16: return launch_general<__half, float>(mode, a, s);
    case DT_F32: return launch_general<float, float>(mode, a, s);
    case DT_F64: return launch_general<double, double>(mode, a, s);
  }
  gbh::set_error("gb_attn_general: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}
