// grouped_gemm.cu - one launch for the feed-forward layers of all experts of a mixture: rows (token, choice) grouped
// by expert, each group multiplied by its own weight matrix.
//
//   C[out_row(s), n] = act( sum_k A[in_row(s), k] * W[e(s)][n, k] )        for s in offsets[e] .. offsets[e+1]
//
// `sorted_pair[s]` = token * top + choice.  The up projection reads the token's row (in_row = pair / top) and writes row s;
// the down projection reads row s and writes row `pair`, so that the caller's weighted sum over a token's choices reads
// them in a fixed order.  Inputs are bf16 or float, products accumulate in float.  A tile never mixes two experts:
// tile y of the grid is mapped to (expert, row block) by walking the group sizes, and tiles beyond the last group exit.
#include "common.cuh"

namespace b2 {

template <typename T> __device__ __forceinline__ float gg_to_f(T v);
template <> __device__ __forceinline__ float gg_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float gg_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T gg_from_f(float v);
template <> __device__ __forceinline__ float gg_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gg_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 16, GG_THREADS = 256;

template <typename T, int ACT /* 0 none, 1 squared ReLU */>
__global__ void __launch_bounds__(GG_THREADS)
grouped_gemm_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W /* [E, N, K] */, T* __restrict__ C, int64_t ldc,
                    const int32_t* __restrict__ offsets, const int32_t* __restrict__ sorted_pair, int E, int N, int K, int top,
                    int in_by_token, int out_by_pair) {
  __shared__ __align__(16) float As[GG_BK][GG_BM + 4];
  __shared__ __align__(16) float Ws[GG_BK][GG_BN + 4];
  __shared__ int in_rows[GG_BM], out_rows[GG_BM];
  // which expert and row block
  int ty = blockIdx.y, e = 0, seg0 = 0, seg1 = 0;
  for (; e < E; ++e) {
    seg0 = offsets[e];
    seg1 = offsets[e + 1];
    const int nt = (seg1 - seg0 + GG_BM - 1) / GG_BM;
    if (ty < nt) break;
    ty -= nt;
  }
  if (e >= E) return;
  const int m0 = seg0 + ty * GG_BM, n0 = blockIdx.x * GG_BN;
  const int tid = threadIdx.x;
  if (tid < GG_BM) {
    const int s = m0 + tid;
    int ir = -1, orow = -1;
    if (s < seg1) {
      const int pair = sorted_pair[s];
      ir = in_by_token ? pair / top : s;
      orow = out_by_pair ? pair : s;
    }
    in_rows[tid] = ir;
    out_rows[tid] = orow;
  }
  __syncthreads();
  const T* We = W + static_cast<size_t>(e) * N * K;
  const int lr = tid >> 2, lk = (tid & 3) * 4;         // loader: row lr, 4 consecutive k
  const int a_row = in_rows[lr];
  const int w_row = n0 + lr;
  const int cx = tid & 15, cy = tid >> 4;              // compute: rows cy*4.., columns cx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_row >= 0 && k < K) ? gg_to_f(A[static_cast<int64_t>(a_row) * lda + k]) : 0.f;
      Ws[lk + i][lr] = (w_row < N && k < K) ? gg_to_f(We[static_cast<size_t>(w_row) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GG_BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][cy * 4]);
      const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][cx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int orow = out_rows[cy * 4 + i];
    if (orow < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + cx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (ACT == 1) { v = fmaxf(v, 0.f); v = v * v; }
      C[static_cast<int64_t>(orow) * ldc + n] = gg_from_f<T>(v);
    }
  }
}

// ------------------------------------------------------------------ bf16 on the tensor cores
// 128 x 128 output tile per CTA, K walked in 64-wide slices through a three-stage ring of 16-byte asynchronous copies
// (rows of A are gathered through `in_rows`; rows of W beyond N and slices beyond K arrive as zeros).  Shared rows are
// padded to 144 bytes, which puts the eight rows of an ldmatrix phase into eight different 16-byte bank groups.  Eight
// warps as 2 (rows) x 4 (columns), a warp owns 64 x 32 as 4 x 4 m16n8k16 accumulators in float.  A 16-row block with
// no row of the group is skipped by its warp, so a decode step (a handful of rows per expert) spends its time
// streaming W once, not multiplying zeros; rows of A beyond the group are not even loaded, since an output row
// depends on its own input row only and those outputs are never stored.
// For decode-sized groups the same kernel runs with 32-row tiles (one row of eight warps, 32 x 16 each) and a four-stage
// ring: the A tile is small, so more bytes of W are in flight per SM.
constexpr int GM_BN = 128, GM_BK = 64, GM_THREADS = 256, GM_LD = GM_BK + 8;
constexpr int GM_CPR = GM_BK / 8;                  // 16-byte chunks per tile row
constexpr int GM_RPP = GM_THREADS / GM_CPR;        // tile rows one pass of the CTA's loader covers
constexpr int GM_PASSES = 128 / GM_RPP;
template <int BM> struct GmShape {
  static constexpr int STAGES = BM == 128 ? 3 : 4;
  static constexpr int WARPS_M = BM == 128 ? 2 : 1, WARPS_N = 8 / WARPS_M;
  static constexpr int MT = BM / WARPS_M / 16, NT = GM_BN / WARPS_N / 8;
  static constexpr size_t SMEM = sizeof(__nv_bfloat16) * STAGES * (BM + GM_BN) * GM_LD + sizeof(int) * 2 * BM;
};

template <int GM_BM, int ACT>
__global__ void __launch_bounds__(GM_THREADS, 2)
grouped_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, const __nv_bfloat16* __restrict__ W,
                        __nv_bfloat16* __restrict__ C, int64_t ldc, const int32_t* __restrict__ offsets,
                        const int32_t* __restrict__ sorted_pair, int E, int N, int K, int top, int in_by_token, int out_by_pair,
                        int paired_store) {
  using S = GmShape<GM_BM>;
  constexpr int GM_STAGES = S::STAGES, MT = S::MT, NT = S::NT;
  extern __shared__ __align__(16) unsigned char gm_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gm_smem);       // [STAGES][BM][LD]
  __nv_bfloat16* Ws = As + GM_STAGES * GM_BM * GM_LD;                  // [STAGES][BN][LD]
  int* in_rows = reinterpret_cast<int*>(Ws + GM_STAGES * GM_BN * GM_LD);
  int* out_rows = in_rows + GM_BM;
  int ty = blockIdx.y, e = 0, seg0 = 0, seg1 = 0;
  for (; e < E; ++e) {
    seg0 = offsets[e];
    seg1 = offsets[e + 1];
    const int nt = (seg1 - seg0 + GM_BM - 1) / GM_BM;
    if (ty < nt) break;
    ty -= nt;
  }
  if (e >= E) return;
  const int m0 = seg0 + ty * GM_BM, n0 = blockIdx.x * GM_BN;
  const int rows = min(GM_BM, seg1 - m0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < GM_BM) {
    const int s = m0 + tid;
    int ir = -1, orow = -1;
    if (tid < rows) {
      const int pair = sorted_pair[s];
      ir = in_by_token ? pair / top : s;
      orow = out_by_pair ? pair : s;
    }
    in_rows[tid] = ir;
    out_rows[tid] = orow;
  }
  __syncthreads();
  const __nv_bfloat16* We = W + static_cast<size_t>(e) * N * K;
  // loader: pass i covers tile rows GM_RPP * i + tid / GM_CPR, 8 columns from (tid % GM_CPR) * 8
  int a_row[GM_PASSES], w_row[GM_PASSES];
#pragma unroll
  for (int i = 0; i < GM_PASSES; ++i) {
    const int r = GM_RPP * i + tid / GM_CPR;
    a_row[i] = r < GM_BM ? in_rows[r] : -1;
    w_row[i] = n0 + r < N ? n0 + r : -1;
  }
  const int ck = (tid % GM_CPR) * 8;
  const int nk = (K + GM_BK - 1) / GM_BK;
  auto load = [&](int stage, int kt) {
    const int k = kt * GM_BK + ck;
#pragma unroll
    for (int i = 0; i < GM_PASSES; ++i) {
      const int r = GM_RPP * i + tid / GM_CPR;
      if (a_row[i] >= 0)
        cp_async_16(As + (stage * GM_BM + r) * GM_LD + ck, A + static_cast<int64_t>(a_row[i]) * lda + (k < K ? k : 0), k < K);
      const bool okw = w_row[i] >= 0 && k < K;
      cp_async_16(Ws + (stage * GM_BN + r) * GM_LD + ck, We + (okw ? static_cast<size_t>(w_row[i]) * K + k : 0), okw);
    }
  };
  const int wm = warp / S::WARPS_N, wn = warp % S::WARPS_N;
  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
#pragma unroll
  for (int s = 0; s < GM_STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<GM_STAGES - 2>();
    __syncthreads();                                   // slice kt has landed; the stage of slice kt - 1 is free
    if (kt + GM_STAGES - 1 < nk) load((kt + GM_STAGES - 1) % GM_STAGES, kt + GM_STAGES - 1);
    cp_async_commit();
    const __nv_bfloat16* Ast = As + (kt % GM_STAGES) * GM_BM * GM_LD;
    const __nv_bfloat16* Wst = Ws + (kt % GM_STAGES) * GM_BN * GM_LD;
#pragma unroll
    for (int ks = 0; ks < GM_BK / 16; ++ks) {
      uint32_t b[NT / 2][4];
#pragma unroll
      for (int np = 0; np < NT / 2; ++np)
        ldsm_x4(b[np][0], b[np][1], b[np][2], b[np][3],
                Wst + (wn * NT * 8 + np * 16 + (lane >> 4) * 8 + (lane & 7)) * GM_LD + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (wm * MT * 16 + mt * 16 >= rows) continue;  // warp-uniform
        uint32_t a[4];
        ldsm_x4(a[0], a[1], a[2], a[3], Ast + (wm * MT * 16 + mt * 16 + (lane & 15)) * GM_LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[mt][nt], a, b[nt >> 1][(nt & 1) * 2], b[nt >> 1][(nt & 1) * 2 + 1]);
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * MT * 16 + mt * 16 + (lane >> 2) + 8 * half;
      const int orow = out_rows[r];
      if (orow < 0) continue;
      __nv_bfloat16* crow = C + static_cast<int64_t>(orow) * ldc;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = n0 + wn * NT * 8 + nt * 8 + 2 * (lane & 3);
        float v0 = acc[mt][nt][2 * half], v1 = acc[mt][nt][2 * half + 1];
        if (ACT == 1) { v0 = fmaxf(v0, 0.f); v0 *= v0; v1 = fmaxf(v1, 0.f); v1 *= v1; }
        if (paired_store && n + 1 < N) {
          *reinterpret_cast<uint32_t*>(crow + n) = pack_bf16(v0, v1);
        } else {
          if (n < N) crow[n] = __float2bfloat16_rn(v0);
          if (n + 1 < N) crow[n + 1] = __float2bfloat16_rn(v1);
        }
      }
    }
  }
}

template <int BM, int ACT>
static cudaError_t launch_grouped_mma(int n_pairs, cudaStream_t st, const void* a, int64_t lda, const void* w, void* c, int64_t ldc,
                                      const int32_t* offsets, const int32_t* sorted_pair, int E, int N, int K, int top,
                                      int in_by_token, int out_by_pair) {
  auto kern = grouped_gemm_mma_kernel<BM, ACT>;
  constexpr size_t GM_SMEM = GmShape<BM>::SMEM;
  const dim3 grid((N + GM_BN - 1) / GM_BN, (n_pairs + BM - 1) / BM + E);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GM_SMEM));
  if (e != cudaSuccess) return e;
  const int paired = (ldc % 2 == 0) && (reinterpret_cast<uintptr_t>(c) % 4 == 0);
  kern<<<grid, GM_THREADS, GM_SMEM, st>>>(static_cast<const __nv_bfloat16*>(a), lda, static_cast<const __nv_bfloat16*>(w),
                                          static_cast<__nv_bfloat16*>(c), ldc, offsets, sorted_pair, E, N, K, top, in_by_token,
                                          out_by_pair, paired);
  return cudaSuccess;
}

}  // namespace b2

extern "C" int b2tts_grouped_gemm(const void* a, int64_t lda, const void* w, void* c, int64_t ldc, const int32_t* offsets,
                                  const int32_t* sorted_pair, int n_pairs, int experts, int n, int k, int top, int in_by_token,
                                  int out_by_pair, int act, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(n_pairs >= 0 && experts > 0 && n > 0 && k > 0 && top > 0, B2TTS_EINVAL, "grouped_gemm: bad sizes");
  B2_REQUIRE(dtype == B2TTS_DTYPE_BF16 || dtype == B2TTS_DTYPE_F32, B2TTS_EINVAL, "grouped_gemm: dtype %d", dtype);
  B2_REQUIRE(act == 0 || act == 1, B2TTS_EINVAL, "grouped_gemm: act %d", act);
  if (n_pairs == 0) return B2TTS_OK;
  B2_REQUIRE(a && w && c && offsets && sorted_pair, B2TTS_EINVAL, "grouped_gemm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // bf16 with 16-byte rows: the tensor-core kernel; float (true 32-bit products) and odd sizes: the plain one
  if (dtype == B2TTS_DTYPE_BF16 && k % 8 == 0 && lda % 8 == 0 && aligned16(a) && aligned16(w)) {
    // groups of a decode step (16 rows per expert on average, or fewer): the 32-row shape
    const bool small = n_pairs <= 16 * experts;
#define GM_GO(BM, ACT) launch_grouped_mma<BM, ACT>(n_pairs, st, a, lda, w, c, ldc, offsets, sorted_pair, experts, n, k, top, in_by_token, out_by_pair)
    cudaError_t e = small ? (act ? GM_GO(32, 1) : GM_GO(32, 0)) : (act ? GM_GO(128, 1) : GM_GO(128, 0));
#undef GM_GO
    if (e != cudaSuccess) return cuda_fail(e, "grouped_gemm (tensor)");
    B2_CHECK_LAUNCH("grouped_gemm (tensor)");
    return B2TTS_OK;
  }
  const dim3 grid((n + GG_BN - 1) / GG_BN, (n_pairs + GG_BM - 1) / GG_BM + experts);
#define GG_GO(T, ACT) grouped_gemm_kernel<T, ACT><<<grid, GG_THREADS, 0, st>>>(static_cast<const T*>(a), lda, static_cast<const T*>(w), \
      static_cast<T*>(c), ldc, offsets, sorted_pair, experts, n, k, top, in_by_token, out_by_pair)
  if (dtype == B2TTS_DTYPE_BF16) { if (act) GG_GO(__nv_bfloat16, 1); else GG_GO(__nv_bfloat16, 0); }
  else { if (act) GG_GO(float, 1); else GG_GO(float, 0); }
#undef GG_GO
  B2_CHECK_LAUNCH("grouped_gemm");
  return B2TTS_OK;
}
