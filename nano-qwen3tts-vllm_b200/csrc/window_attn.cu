// window_attn.cu - sliding-window attention with un-normalised sigmoid weights and a logarithmic distance bias over the
// paged K/V cache, for prompt portions and single decoded tokens in one launch.
//
//   out[i, h] = sum over j with 0 <= i - j < window of  sigmoid(q_ih . k_jg * scale - r1_h * ln(1 + r2_h * (i - j)) + pb_h) * v_jg
//
// with g = h / (heads / kv_heads).  There is no softmax, hence no running maximum and no rescaling: a key tile only adds
// to the accumulator.  Scores, weights and the accumulator are float for both cache types (bf16 or float).
//
// One CTA owns 32 (query token, head of the group) rows of ONE sequence and ONE key/value head, so the K/V tile it stages in
// shared memory serves every query head of the group.  Keys are read through the block table: the step's own tokens were
// written to the cache by the preceding kernel, so a portion in the middle of a prompt and a decoded token look the same.
#include <math.h>

#include "common.cuh"

namespace b2 {

template <typename T> __device__ __forceinline__ float wa_to_f(T v);
template <> __device__ __forceinline__ float wa_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float wa_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T wa_from_f(float v);
template <> __device__ __forceinline__ float wa_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 wa_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int WA_ROWS = 32;      // (token, head-in-group) rows per CTA
constexpr int WA_WARPS = 4;
constexpr int WA_RPW = WA_ROWS / WA_WARPS;
constexpr int WA_BK = 32;        // keys per tile = one per lane in the score phase

template <typename T, int DVL>
__global__ void __launch_bounds__(WA_WARPS * 32)
window_sigmoid_attn_kernel(const T* __restrict__ q /* [n, H*d] */, const T* __restrict__ k_cache /* [slots, G*d] */,
                           const T* __restrict__ v_cache /* [slots, G*dv] */, T* __restrict__ out /* [n, H*dv] */,
                           const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                           const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_tables, int bt_stride,
                           const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb,
                           int H, int G, int d, int dv, int page, int window, float scale) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.z, g = blockIdx.y;
  const int len = seq_len[b];
  const int rep = H / G;
  const int row0 = blockIdx.x * WA_ROWS;
  if (len <= 0) {
    // a padding row of a captured decode step: its one output row is zeroed so that nothing undefined flows on
    if (blockIdx.x == 0)
      for (int c = threadIdx.x; c < rep * dv; c += blockDim.x)
        out[static_cast<size_t>(seq_start[b]) * H * dv + g * rep * dv + c] = wa_from_f<T>(0.f);
    return;
  }
  if (row0 >= len * rep) return;
  const int d4 = (d + 3) & ~3, kstride = d4 + 4;
  float* qs = smem;                                  // [ROWS][d4]
  float* ks = qs + WA_ROWS * d4;                     // [BK][d4 + 4]
  float* vs = ks + WA_BK * kstride;                  // [BK][dv]
  float* ws = vs + WA_BK * dv;                       // [ROWS][BK + 1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = seq_start[b], pos0 = seq_pos0[b];
  const int32_t* bt = block_tables + static_cast<size_t>(b) * bt_stride;

  // stage the query rows (zero rows beyond the sequence's portion and zero padding columns)
  for (int idx = tid; idx < WA_ROWS * d4; idx += blockDim.x) {
    const int r = idx / d4, c = idx % d4;
    const int rg = row0 + r, t = rg / rep, hr = rg % rep;
    float v = 0.f;
    if (t < len && c < d) v = wa_to_f(q[static_cast<size_t>(start + t) * H * d + (g * rep + hr) * d + c]);
    qs[idx] = v;
  }
  const int t_lo = row0 / rep;
  const int t_hi = min(len - 1, (row0 + WA_ROWS - 1) / rep);
  const int j_lo = max(0, pos0 + t_lo - window + 1), j_hi = pos0 + t_hi;

  // this warp's rows
  int my_p[WA_RPW], my_h[WA_RPW];
  float my_r1[WA_RPW], my_r2[WA_RPW], my_pb[WA_RPW];
  bool warp_live = false;
#pragma unroll
  for (int i = 0; i < WA_RPW; ++i) {
    const int rg = row0 + warp * WA_RPW + i, t = rg / rep, hr = rg % rep;
    const bool ok = t < len;
    my_p[i] = ok ? pos0 + t : -1;
    my_h[i] = g * rep + hr;
    my_r1[i] = ok ? r1[my_h[i]] : 0.f;
    my_r2[i] = ok ? r2[my_h[i]] : 0.f;
    my_pb[i] = ok ? pb[my_h[i]] : 0.f;
    warp_live |= ok;
  }
  float acc[WA_RPW][DVL];
#pragma unroll
  for (int i = 0; i < WA_RPW; ++i)
#pragma unroll
    for (int l = 0; l < DVL; ++l) acc[i][l] = 0.f;

  for (int j0 = j_lo; j0 <= j_hi; j0 += WA_BK) {
    __syncthreads();                                 // the previous tile is consumed (and qs is written, first time)
    for (int idx = tid; idx < WA_BK * d4; idx += blockDim.x) {
      const int jj = idx / d4, c = idx % d4, j = j0 + jj;
      float v = 0.f;
      if (j <= j_hi && c < d) {
        const size_t slot = static_cast<size_t>(bt[j / page]) * page + j % page;
        v = wa_to_f(k_cache[slot * G * d + g * d + c]);
      }
      ks[jj * kstride + c] = v;
    }
    for (int idx = tid; idx < WA_BK * dv; idx += blockDim.x) {
      const int jj = idx / dv, c = idx % dv, j = j0 + jj;
      float v = 0.f;
      if (j <= j_hi) {
        const size_t slot = static_cast<size_t>(bt[j / page]) * page + j % page;
        v = wa_to_f(v_cache[slot * G * dv + g * dv + c]);
      }
      vs[idx] = v;
    }
    __syncthreads();
    if (!warp_live) continue;
    // scores: lane = key
    float s[WA_RPW];
#pragma unroll
    for (int i = 0; i < WA_RPW; ++i) s[i] = 0.f;
    const float4* kr = reinterpret_cast<const float4*>(ks + lane * kstride);
    for (int c4 = 0; c4 < d4 / 4; ++c4) {
      const float4 kv = kr[c4];
#pragma unroll
      for (int i = 0; i < WA_RPW; ++i) {
        const float4 qv = reinterpret_cast<const float4*>(qs + (warp * WA_RPW + i) * d4)[c4];
        s[i] = fmaf(qv.x, kv.x, s[i]);
        s[i] = fmaf(qv.y, kv.y, s[i]);
        s[i] = fmaf(qv.z, kv.z, s[i]);
        s[i] = fmaf(qv.w, kv.w, s[i]);
      }
    }
    const int j = j0 + lane;
#pragma unroll
    for (int i = 0; i < WA_RPW; ++i) {
      const int dist = my_p[i] - j;
      float w = 0.f;
      if (my_p[i] >= 0 && j <= j_hi && dist >= 0 && dist < window) {
        const float z = s[i] * scale - my_r1[i] * log1pf(my_r2[i] * static_cast<float>(dist)) + my_pb[i];
        w = 1.0f / (1.0f + expf(-z));
      }
      ws[(warp * WA_RPW + i) * (WA_BK + 1) + lane] = w;
    }
    __syncwarp();
    // out += weights x values: lane = value column
    for (int jj = 0; jj < WA_BK; ++jj) {
      float vv[DVL];
#pragma unroll
      for (int l = 0; l < DVL; ++l) vv[l] = (lane + 32 * l < dv) ? vs[jj * dv + lane + 32 * l] : 0.f;
#pragma unroll
      for (int i = 0; i < WA_RPW; ++i) {
        const float w = ws[(warp * WA_RPW + i) * (WA_BK + 1) + jj];
#pragma unroll
        for (int l = 0; l < DVL; ++l) acc[i][l] = fmaf(w, vv[l], acc[i][l]);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < WA_RPW; ++i) {
    if (my_p[i] < 0) continue;
    const int t = my_p[i] - pos0;
    T* o = out + static_cast<size_t>(start + t) * H * dv + my_h[i] * dv;
#pragma unroll
    for (int l = 0; l < DVL; ++l)
      if (lane + 32 * l < dv) o[lane + 32 * l] = wa_from_f<T>(acc[i][l]);
  }
}

template <typename T, int DVL>
static cudaError_t launch_window_attn(dim3 grid, size_t smem, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                      const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                      const int32_t* bt, int bt_stride, const float* r1, const float* r2, const float* pb, int H,
                                      int G, int d, int dv, int page, int window, float scale) {
  auto kern = window_sigmoid_attn_kernel<T, DVL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, WA_WARPS * 32, smem, st>>>(static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc),
                                          static_cast<T*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb, H, G, d,
                                          dv, page, window, scale);
  return cudaSuccess;
}

}  // namespace b2

extern "C" int b2tts_window_sigmoid_attn(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                         const int32_t* block_tables, int bt_stride, const float* r1, const float* r2,
                                         const float* pb, int n_seqs, int max_new, int heads, int kv_heads, int dim, int vdim,
                                         int page, int window, float scale, int dtype, void* stream) {
  using namespace b2;
  B2_REQUIRE(n_seqs >= 0 && max_new >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 &&
             page > 0 && window > 0 && bt_stride > 0, B2TTS_EINVAL, "window_sigmoid_attn: bad sizes");
  B2_REQUIRE(dtype == B2TTS_DTYPE_BF16 || dtype == B2TTS_DTYPE_F32, B2TTS_EINVAL, "window_sigmoid_attn: dtype %d", dtype);
  B2_REQUIRE(vdim <= 256, B2TTS_EUNSUPPORTED, "window_sigmoid_attn: value size %d > 256", vdim);
  if (n_seqs == 0 || max_new == 0) return B2TTS_OK;
  B2_REQUIRE(q && k_cache && v_cache && out && seq_start && seq_pos0 && seq_len && block_tables && r1 && r2 && pb, B2TTS_EINVAL,
             "window_sigmoid_attn: null pointer");
  const int rep = heads / kv_heads;
  const int d4 = (dim + 3) & ~3;
  const size_t smem = sizeof(float) * (static_cast<size_t>(WA_ROWS) * d4 + WA_BK * (d4 + 4) + static_cast<size_t>(WA_BK) * vdim +
                                       WA_ROWS * (WA_BK + 1));
  B2_REQUIRE(smem <= 200 * 1024, B2TTS_EUNSUPPORTED, "window_sigmoid_attn: head size %d needs %zu bytes of shared memory", dim, smem);
  const dim3 grid((static_cast<unsigned>(max_new) * rep + WA_ROWS - 1) / WA_ROWS, kv_heads, n_seqs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int dvl = (vdim + 31) / 32;
  cudaError_t e;
#define WA_GO(T, L) e = launch_window_attn<T, L>(grid, smem, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len, block_tables, \
                                                 bt_stride, r1, r2, pb, heads, kv_heads, dim, vdim, page, window, scale)
  if (dtype == B2TTS_DTYPE_BF16) {
    if (dvl <= 1) WA_GO(__nv_bfloat16, 1); else if (dvl <= 2) WA_GO(__nv_bfloat16, 2); else if (dvl <= 4) WA_GO(__nv_bfloat16, 4); else WA_GO(__nv_bfloat16, 8);
  } else {
    if (dvl <= 1) WA_GO(float, 1); else if (dvl <= 2) WA_GO(float, 2); else if (dvl <= 4) WA_GO(float, 4); else WA_GO(float, 8);
  }
#undef WA_GO
  if (e != cudaSuccess) return cuda_fail(e, "window_sigmoid_attn");
  B2_CHECK_LAUNCH("window_sigmoid_attn");
  return B2TTS_OK;
}
