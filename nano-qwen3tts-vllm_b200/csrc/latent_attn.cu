// latent_attn.cu - attention over a paged cache of LATENTS: every cached row is [c (r numbers) | kr (dr numbers)], one
// row per token shared by all heads.  Head h's key is [W_uk,h c | kr] and its value W_uv,h c; both expansions are moved
// out of the loop over keys: the caller multiplies the un-rotated query part by W_uk,h^T once ("absorbed" query
// ql [r]) and applies W_uv,h to the attention-weighted sum of latents afterwards, so that the kernel is multi-query
// attention with key [c | kr] and value c:
//
//   s_ij = scale * (ql_i . c_j + rot(qr_i) . kr_j),   j visible from i:  0 <= i - j (< window, if window > 0)
//   o_i  = sum_j exp(s_ij - m) c_j / (exp(sink_h - m) + sum_j exp(s_ij - m))          (a sink: a slot with no key or value)
//
// The rotated query part is turned here (pairs (2k, 2k+1), angle position * freq[k], cos and sin times rot_mult); the
// keys were turned when they were written.  Scores, weights, maxima and sums are float.  One launch serves a mixed step:
// rows of prompt portions and single decoded tokens, each reading its keys through its sequence's block table.
#include <math.h>

#include "common.cuh"

namespace b2 {
namespace lat {

template <typename T> __device__ __forceinline__ float a_to_f(T v);
template <> __device__ __forceinline__ float a_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float a_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T a_from_f(float v);
template <> __device__ __forceinline__ float a_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 a_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct LatentAttnArgs {
  const void* ql; int64_t ql_tok, ql_head;      // absorbed queries [.., r]
  const void* qr; int64_t qr_tok, qr_head;      // un-rotated rotary query parts [.., dr]
  const void* cache;                            // [pages * page, r + dr]
  void* out; int64_t o_tok, o_head;             // weighted latent sums [.., r]
  const float* sink;                            // [H]
  const float* freq; float rot_mult; int rot_dims;
  const int32_t *seq_start, *seq_pos0, *seq_len, *block_tables; int64_t bt_stride;
  int n_seqs, max_new, H, r, dr, page, window;
  float scale;
};

// ------------------------------------------------------------------ plain kernel (any size, bf16 or float)
// One warp per (token, head).  A batch of 32 keys: lane l scores key l (dot product over the whole row, the query in
// shared memory as floats), then the lanes turn to the latent's coordinates and add the 32 weighted rows.
constexpr int LA_WARPS = 4;
constexpr int LA_MAX_R_PER_LANE = 32;           // latents up to 1024 numbers

template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attn_kernel(const LatentAttnArgs a) {
  extern __shared__ float q_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y;
  const int len = a.seq_len[b];
  const int row = blockIdx.x * LA_WARPS + warp;
  const int tl = row / a.H, h = row % a.H;
  if (tl >= len) return;
  const int Dk = a.r + a.dr;
  float* q = q_smem + warp * Dk;
  const int tok = a.seq_start[b] + tl;
  const int pos = a.seq_pos0[b] + tl;
  const T* ql = static_cast<const T*>(a.ql) + tok * a.ql_tok + h * a.ql_head;
  const T* qr = static_cast<const T*>(a.qr) + tok * a.qr_tok + h * a.qr_head;
  for (int c = lane; c < a.r; c += 32) q[c] = a_to_f(ql[c]) * a.scale;
  for (int i = lane; i < (a.dr + 1) / 2; i += 32) {
    const int c0 = 2 * i, c1 = 2 * i + 1;
    const float u = a_to_f(qr[c0]);
    const float v = c1 < a.dr ? a_to_f(qr[c1]) : 0.f;
    if (c1 < a.rot_dims) {
      float sn, cs;
      sincosf(static_cast<float>(pos) * a.freq[i], &sn, &cs);
      sn *= a.rot_mult; cs *= a.rot_mult;
      q[a.r + c0] = (u * cs - v * sn) * a.scale;
      q[a.r + c1] = (v * cs + u * sn) * a.scale;
    } else {
      q[a.r + c0] = u * a.scale;
      if (c1 < a.dr) q[a.r + c1] = v * a.scale;
    }
  }
  __syncwarp();
  const int32_t* bt = a.block_tables + b * a.bt_stride;
  const T* cache = static_cast<const T*>(a.cache);
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  float m = a.sink[h], l = 1.0f;                 // the sink: exp(sink - m) with m = sink
  float o[LA_MAX_R_PER_LANE];
#pragma unroll
  for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) o[i] = 0.f;
  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool ok = j <= pos;
    size_t slot = 0;
    float s = -INFINITY;
    if (ok) {
      slot = static_cast<size_t>(bt[j / a.page]) * a.page + j % a.page;
      const T* kr = cache + slot * Dk;
      float acc = 0.f;
      for (int c = 0; c < Dk; ++c) acc += q[c] * a_to_f(kr[c]);
      s = acc;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float alpha = expf(m - mn);
    const float p = ok ? expf(s - mn) : 0.f;
    l = l * alpha + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) o[i] *= alpha;
    const int nk = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const size_t sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vr = cache + sj * Dk;
#pragma unroll
      for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) {
        const int c = i * 32 + lane;
        if (c < a.r) o[i] += pj * a_to_f(vr[c]);
      }
    }
  }
  T* orow = static_cast<T*>(a.out) + tok * a.o_tok + h * a.o_head;
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < LA_MAX_R_PER_LANE; ++i) {
    const int c = i * 32 + lane;
    if (c < a.r) orow[c] = a_from_f<T>(o[i] * inv);
  }
}

}  // namespace lat
}  // namespace b2

extern "C" int b2tts_latent_attn(const void* ql, int64_t ql_tok, int64_t ql_head, const void* qr, int64_t qr_tok, int64_t qr_head,
                                 const void* cache, void* out, int64_t o_tok, int64_t o_head, const float* sink, const float* freq,
                                 float rot_mult, int rot_dims, const int32_t* seq_start, const int32_t* seq_pos0,
                                 const int32_t* seq_len, const int32_t* block_tables, int64_t bt_stride, int n_seqs, int max_new,
                                 int heads, int kv_rank, int rot_dim, int page, int window, float scale, int dtype, int path,
                                 void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(n_seqs >= 0 && max_new >= 0 && heads > 0 && kv_rank > 0 && rot_dim >= 0 && page > 0 && window >= 0, B2TTS_EINVAL,
             "latent_attn: bad sizes");
  B2_REQUIRE(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0, B2TTS_EINVAL, "latent_attn: rot_dims %d of %d", rot_dims, rot_dim);
  B2_REQUIRE(dtype == B2TTS_DTYPE_BF16 || dtype == B2TTS_DTYPE_F32, B2TTS_EINVAL, "latent_attn: dtype %d", dtype);
  B2_REQUIRE(kv_rank <= 32 * LA_MAX_R_PER_LANE, B2TTS_EUNSUPPORTED, "latent_attn: latent size %d > %d", kv_rank, 32 * LA_MAX_R_PER_LANE);
  if (n_seqs == 0 || max_new == 0) return B2TTS_OK;
  B2_REQUIRE(ql && cache && out && sink && seq_start && seq_pos0 && seq_len && block_tables && (rot_dim == 0 || qr) &&
             (rot_dims == 0 || freq), B2TTS_EINVAL, "latent_attn: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LatentAttnArgs a{ql, ql_tok, ql_head, qr, qr_tok, qr_head, cache, out, o_tok, o_head, sink, freq, rot_mult, rot_dims,
                   seq_start, seq_pos0, seq_len, block_tables, bt_stride, n_seqs, max_new, heads, kv_rank, rot_dim, page, window, scale};
  (void)path;
  const size_t smem = static_cast<size_t>(LA_WARPS) * (kv_rank + rot_dim) * sizeof(float);
  B2_REQUIRE(smem <= 48 * 1024, B2TTS_EUNSUPPORTED, "latent_attn: key size %d too large", kv_rank + rot_dim);
  const dim3 grid((static_cast<unsigned>(max_new) * heads + LA_WARPS - 1) / LA_WARPS, n_seqs);
  if (dtype == B2TTS_DTYPE_BF16) latent_attn_kernel<__nv_bfloat16><<<grid, LA_WARPS * 32, smem, st>>>(a);
  else latent_attn_kernel<float><<<grid, LA_WARPS * 32, smem, st>>>(a);
  B2_CHECK_LAUNCH("latent_attn");
  return B2TTS_OK;
}
