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
  const dim3 grid((n + GG_BN - 1) / GG_BN, (n_pairs + GG_BM - 1) / GG_BM + experts);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define GG_GO(T, ACT) grouped_gemm_kernel<T, ACT><<<grid, GG_THREADS, 0, st>>>(static_cast<const T*>(a), lda, static_cast<const T*>(w), \
      static_cast<T*>(c), ldc, offsets, sorted_pair, experts, n, k, top, in_by_token, out_by_pair)
  if (dtype == B2TTS_DTYPE_BF16) { if (act) GG_GO(__nv_bfloat16, 1); else GG_GO(__nv_bfloat16, 0); }
  else { if (act) GG_GO(float, 1); else GG_GO(float, 0); }
#undef GG_GO
  B2_CHECK_LAUNCH("grouped_gemm");
  return B2TTS_OK;
}
