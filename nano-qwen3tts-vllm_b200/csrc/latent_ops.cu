// latent_ops.cu - per-row kernels of decoders whose sublayers read the 32-bit residual stream itself and whose output is
// normalised before it is added ("norm on the output"):
//   scaled token embedding; token shift (a per-channel blend with the previous token's row, carried between steps in a
//   state slot); the preparation of a latent-attention step (RMS norm of the query latent, RMS norm of the key/value
//   latent and pair rotation of the shared key part, both written straight into the paged cache); the gate of the
//   attention output; the residual update x += w * group_rms_norm(y) with the weighted sum over experts folded in; the
//   final norm on gathered rows; the xIELU activation and the gated SiLU product.
//
// Activations are `T` = bf16 (serving) or float (the all-32-bit mode).  The residual stream, every norm, every angle and
// every per-channel constant are float in both.  Nothing allocates or synchronises; every launch is graph-capturable.
#include <math.h>

#include <algorithm>

#include "common.cuh"

namespace b2 {
namespace lat {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int ROW_THREADS = 256;

// sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ------------------------------------------------------------------ x = embed[token] * scale
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
embed_scale_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, float* __restrict__ x, int cols, int vocab,
                   float scale) {
  const size_t row = blockIdx.x;
  const int tok = min(max(tokens[row], 0), vocab - 1);
  const T* er = embed + static_cast<size_t>(tok) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) x[row * cols + c] = to_f(er[c]) * scale;
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&lo);
  v.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

// ------------------------------------------------------------------ token shift
// out[t] = x[t] + (prev - x[t]) * mu, prev = the same layer's input row of the previous position: x[t - 1] when that
// position runs in this step, the sequence's state slot when it ran in an earlier step, zero at position 0 (by position:
// a slot is never cleared).  The block of a sequence's FIRST token in the step is the only reader of the slot, and it
// is also the one that then overwrites it with the sequence's LAST row of the step, so no order between blocks matters.
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                   const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_len,
                   const int32_t* __restrict__ seq_slot, T* __restrict__ out, int cols) {
  const size_t t = blockIdx.x;
  const int b = tok_seq[t];
  const int len = seq_len[b];
  T* orow = out + t * cols;
  if (len <= 0) {                                                       // a padding row of a captured step
    for (int c = threadIdx.x; c < cols; c += blockDim.x) orow[c] = from_f<T>(0.f);
    return;
  }
  const int start = seq_start[b];
  const bool first = static_cast<int>(t) == start;
  const int pos = positions[t];
  float* srow = state + static_cast<size_t>(seq_slot[b]) * cols;
  const float* xr = x + t * cols;
  const float* pr = first ? srow : xr - cols;
  const float* last = x + static_cast<size_t>(start + len - 1) * cols;
  if (cols % 4 == 0) {                                                    // rows of whole float4: 16-byte loads, 8- or 16-byte stores
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    const float4* p4 = reinterpret_cast<const float4*>(pr);
    const float4* m4 = reinterpret_cast<const float4*>(mu);
    const float4* l4 = reinterpret_cast<const float4*>(last);
    float4* s4 = reinterpret_cast<float4*>(srow);
    for (int c = threadIdx.x; c < cols / 4; c += blockDim.x) {
      const float4 cur = x4[c], m = m4[c];
      const float4 prev = pos > 0 ? p4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
      store4(orow + 4 * c, cur.x + (prev.x - cur.x) * m.x, cur.y + (prev.y - cur.y) * m.y, cur.z + (prev.z - cur.z) * m.z,
             cur.w + (prev.w - cur.w) * m.w);
      if (first) s4[c] = l4[c];                                           // same thread read s4[c] just above
    }
    return;
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float cur = xr[c];
    const float prev = pos > 0 ? pr[c] : 0.f;
    orow[c] = from_f<T>(cur + (prev - cur) * mu[c]);
    if (first) srow[c] = last[c];                                       // same thread read srow[c] just above
  }
}

// ------------------------------------------------------------------ latent preparation
// u[t] = [ .. | query latent (q_rank) .. | key/value latent (kv_rank) | shared key part (rot_dim) | .. ] is one row of a
// merged projection.  Writes cq[t] = rms_norm(query latent) * wq (if q_rank > 0), and into the cache row slot_mapping[t]:
// [rms_norm(latent) * wkv | rotate(shared key part)].  Pair (2i, 2i+1), i < rot_dims / 2, turns by positions[t] * freq[i];
// cos and sin are multiplied by rot_mult; coordinates from rot_dims on pass unchanged.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ u, int64_t ldu, int q_off, int kv_off, T* __restrict__ cq, const float* __restrict__ wq,
                   const float* __restrict__ wkv, const float* __restrict__ freq, float rot_mult,
                   const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, T* __restrict__ cache,
                   int q_rank, int kv_rank, int rot_dim, int rot_dims, float eps) {
  __shared__ float red[33];
  const size_t t = blockIdx.x;
  const T* ur = u + t * ldu;
  if (q_rank > 0) {
    const T* qr = ur + q_off;
    float ssq = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) { const float v = to_f(qr[c]); ssq += v * v; }
    const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(q_rank) + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq[t * q_rank + c] = from_f<T>(to_f(qr[c]) * inv * wq[c]);
  }
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const T* kr = ur + kv_off;
  T* crow = cache + static_cast<size_t>(slot) * (kv_rank + rot_dim);
  float ssq = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) { const float v = to_f(kr[c]); ssq += v * v; }
  const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(kv_rank) + eps);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) crow[c] = from_f<T>(to_f(kr[c]) * inv * wkv[c]);
  const float p = static_cast<float>(positions[t]);
  for (int i = threadIdx.x; i < rot_dim / 2 + (rot_dim & 1); i += blockDim.x) {
    const int c0 = 2 * i, c1 = 2 * i + 1;
    const float a = to_f(kr[kv_rank + c0]);
    const float b = c1 < rot_dim ? to_f(kr[kv_rank + c1]) : 0.f;
    if (c1 < rot_dims) {
      float sn, cs;
      sincosf(p * freq[i], &sn, &cs);
      sn *= rot_mult; cs *= rot_mult;
      crow[kv_rank + c0] = from_f<T>(a * cs - b * sn);
      crow[kv_rank + c1] = from_f<T>(b * cs + a * sn);
    } else {
      crow[kv_rank + c0] = from_f<T>(a);
      if (c1 < rot_dim) crow[kv_rank + c1] = from_f<T>(b);
    }
  }
}

// ------------------------------------------------------------------ gate of the attention output + head-major -> row-major
// out[t, h * dv + d] = v[h, t, d] (strides given) * sigmoid(gate[t, h * dv + d]); without a gate it is the plain re-layout.
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ v, int64_t v_tok, int64_t v_head, const T* __restrict__ gate, int64_t ldg,
                                  T* __restrict__ out, int n, int H, int dv) {
  const size_t total = static_cast<size_t>(n) * H * dv;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(i % dv);
    const int h = static_cast<int>((i / dv) % H);
    const size_t t = i / (static_cast<size_t>(dv) * H);
    float val = to_f(v[t * v_tok + h * v_head + d]);
    if (gate != nullptr) val *= 1.0f / (1.0f + expf(-to_f(gate[t * ldg + static_cast<size_t>(h) * dv + d])));
    out[i] = from_f<T>(val);
  }
}

// ------------------------------------------------------------------ x += w * group_rms_norm(y)
// y[row] = a[row] (if given) + sum_k zw[row, k] * z[row * top + k] (if given), in float, experts in the order k = 0 ..;
// the row is cut into `groups` equal parts, each divided by its own sqrt(mean(part^2) + eps).  `copy` (optional) receives
// the new x[row] in the activation type: the input of the sublayer that follows.
template <typename T>
__device__ __forceinline__ float sub_out(const T* a, const T* z, const float* zw, int top, size_t row, int cols, int c) {
  float s = 0.f;
  if (a != nullptr) s += to_f(a[row * cols + c]);
  if (z != nullptr) {
    float e = 0.f;
    for (int k = 0; k < top; ++k) e += zw[row * top + k] * to_f(z[(row * top + k) * cols + c]);
    s += e;
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
group_norm_residual_kernel(float* __restrict__ x, const T* __restrict__ a, const T* __restrict__ z, const float* __restrict__ zw,
                           int top, const float* __restrict__ w, int groups, float eps, T* __restrict__ copy, int cols) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const int gs = cols / groups;
  for (int g = 0; g < groups; ++g) {               // one fixed-order block reduction per group: the same bits every run
    float ssq = 0.f;
    for (int c = g * gs + threadIdx.x; c < (g + 1) * gs; c += blockDim.x) {
      const float v = sub_out<T>(a, z, zw, top, row, cols, c);
      ssq += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(gs) + eps);
    for (int c = g * gs + threadIdx.x; c < (g + 1) * gs; c += blockDim.x) {
      const float v = sub_out<T>(a, z, zw, top, row, cols, c);
      const float nx = x[row * cols + c] + v * inv * w[c];
      x[row * cols + c] = nx;
      if (copy != nullptr) copy[row * cols + c] = from_f<T>(nx);
    }
  }
}

// out[i] = group_rms_norm(x[rows[i]]) * w  (the rows whose logits are wanted), or out[i] = T(x[rows[i]]) when w is null
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
gather_group_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, T* __restrict__ out,
                         const float* __restrict__ w, int groups, float eps, int cols) {
  __shared__ float red[33];
  const size_t src = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * cols;
  T* orow = out + static_cast<size_t>(blockIdx.x) * cols;
  if (w == nullptr) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) orow[c] = from_f<T>(xr[c]);
    return;
  }
  const int gs = cols / groups;
  for (int g = 0; g < groups; ++g) {
    float ssq = 0.f;
    for (int c = g * gs + threadIdx.x; c < (g + 1) * gs; c += blockDim.x) ssq += xr[c] * xr[c];
    const float inv = 1.0f / sqrtf(block_sum(ssq, red) / static_cast<float>(gs) + eps);
    for (int c = g * gs + threadIdx.x; c < (g + 1) * gs; c += blockDim.x) orow[c] = from_f<T>(xr[c] * inv * w[c]);
  }
}

// ------------------------------------------------------------------ activations
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// xIELU in place, with an optional bias added first: z > 0: sp(p) z^2 + z/2;  z <= 0: (1/2 + sp(q)) (e^z - 1 - z) + z/2
template <typename T>
__global__ void xielu_kernel(T* __restrict__ y, const T* __restrict__ bias, const float* __restrict__ pq, size_t n, int cols) {
  const float ap = softplus_f(pq[0]), aq = 0.5f + softplus_f(pq[1]);
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float z = to_f(y[i]);
    if (bias != nullptr) z += to_f(bias[i % cols]);
    const float r = z > 0.f ? ap * z * z + 0.5f * z : aq * (expm1f(z) - z) + 0.5f * z;
    y[i] = from_f<T>(r);
  }
}

// y[r, c] = silu(gu[r, c]) * gu[r, ff + c]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ y, size_t rows, int ff) {
  const size_t n = rows * ff;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / ff;
    const int c = static_cast<int>(i % ff);
    const float g = to_f(gu[r * 2 * ff + c]), u = to_f(gu[r * 2 * ff + ff + c]);
    y[i] = from_f<T>(g / (1.0f + expf(-g)) * u);
  }
}

static int flat_grid(size_t n) { return static_cast<int>(std::min<size_t>((n + 255) / 256, 148 * 16)); }

}  // namespace lat
}  // namespace b2

#define LAT_DTYPE_OK(dt) ((dt) == B2TTS_DTYPE_BF16 || (dt) == B2TTS_DTYPE_F32)
#define LAT_DISPATCH(dt, CALL) do { if ((dt) == B2TTS_DTYPE_BF16) { using T = __nv_bfloat16; CALL; } else { using T = float; CALL; } } while (0)

extern "C" int b2tts_embed_scale(const int32_t* tokens, const void* embed, float* x, int rows, int cols, int vocab, float scale,
                                 int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(rows >= 0 && cols > 0 && vocab > 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "embed_scale: rows=%d cols=%d dtype=%d", rows, cols, dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(tokens && embed && x, B2TTS_EINVAL, "embed_scale: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (embed_scale_kernel<T><<<rows, ROW_THREADS, 0, st>>>(tokens, static_cast<const T*>(embed), x, cols, vocab, scale)));
  B2_CHECK_LAUNCH("embed_scale");
  return B2TTS_OK;
}

extern "C" int b2tts_token_shift(const float* x, const float* mu, float* state, const int32_t* tok_seq, const int32_t* positions,
                                 const int32_t* seq_start, const int32_t* seq_len, const int32_t* seq_slot, void* out,
                                 int n_tokens, int cols, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(n_tokens >= 0 && cols > 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "token_shift: n=%d cols=%d dtype=%d", n_tokens, cols, dtype);
  if (n_tokens == 0) return B2TTS_OK;
  B2_REQUIRE(x && mu && state && tok_seq && positions && seq_start && seq_len && seq_slot && out, B2TTS_EINVAL, "token_shift: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (token_shift_kernel<T><<<n_tokens, ROW_THREADS, 0, st>>>(x, mu, state, tok_seq, positions, seq_start, seq_len,
                                                                              seq_slot, static_cast<T*>(out), cols)));
  B2_CHECK_LAUNCH("token_shift");
  return B2TTS_OK;
}

extern "C" int b2tts_latent_prep(const void* u, int64_t ldu, int q_off, int kv_off, void* cq, const float* q_norm_w,
                                 const float* kv_norm_w, const float* freq, float rot_mult, const int32_t* positions,
                                 const int32_t* slot_mapping, void* cache, int n_tokens, int q_rank, int kv_rank, int rot_dim,
                                 int rot_dims, float eps, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(n_tokens >= 0 && q_rank >= 0 && kv_rank > 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0,
             B2TTS_EINVAL, "latent_prep: n=%d q_rank=%d kv_rank=%d rot_dim=%d rot_dims=%d", n_tokens, q_rank, kv_rank, rot_dim, rot_dims);
  B2_REQUIRE(LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "latent_prep: dtype %d", dtype);
  if (n_tokens == 0) return B2TTS_OK;
  B2_REQUIRE(u && kv_norm_w && positions && slot_mapping && cache && (rot_dims == 0 || freq) && (q_rank == 0 || (cq && q_norm_w)),
             B2TTS_EINVAL, "latent_prep: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (latent_prep_kernel<T><<<n_tokens, 128, 0, st>>>(static_cast<const T*>(u), ldu, q_off, kv_off, static_cast<T*>(cq),
      q_norm_w, kv_norm_w, freq, rot_mult, positions, slot_mapping, static_cast<T*>(cache), q_rank, kv_rank, rot_dim, rot_dims, eps)));
  B2_CHECK_LAUNCH("latent_prep");
  return B2TTS_OK;
}

extern "C" int b2tts_gate_heads(const void* v, int64_t v_tok, int64_t v_head, const void* gate, int64_t ldg, void* out, int n,
                                int heads, int vdim, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(n >= 0 && heads > 0 && vdim > 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "gate_heads: n=%d heads=%d vdim=%d", n, heads, vdim);
  if (n == 0) return B2TTS_OK;
  B2_REQUIRE(v && out, B2TTS_EINVAL, "gate_heads: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = flat_grid(static_cast<size_t>(n) * heads * vdim);
  LAT_DISPATCH(dtype, (gate_heads_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(v), v_tok, v_head, static_cast<const T*>(gate), ldg,
                                                                 static_cast<T*>(out), n, heads, vdim)));
  B2_CHECK_LAUNCH("gate_heads");
  return B2TTS_OK;
}

extern "C" int b2tts_group_norm_residual(float* x, const void* a, const void* z, const float* zw, int top, const float* w, int groups,
                                         float eps, void* copy, int rows, int cols, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(rows >= 0 && cols > 0 && top >= 0 && groups > 0 && cols % groups == 0, B2TTS_EINVAL,
             "group_norm_residual: rows=%d cols=%d top=%d groups=%d", rows, cols, top, groups);
  B2_REQUIRE(LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "group_norm_residual: dtype %d", dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(x && w && (a || z) && (!z || (zw && top > 0)), B2TTS_EINVAL, "group_norm_residual: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (group_norm_residual_kernel<T><<<rows, ROW_THREADS, 0, st>>>(x, static_cast<const T*>(a), static_cast<const T*>(z), zw,
      top, w, groups, eps, static_cast<T*>(copy), cols)));
  B2_CHECK_LAUNCH("group_norm_residual");
  return B2TTS_OK;
}

extern "C" int b2tts_gather_group_norm(const float* x, const int32_t* rows_idx, void* out, const float* w, int groups, float eps,
                                       int rows, int cols, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(rows >= 0 && cols > 0 && groups > 0 && cols % groups == 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL,
             "gather_group_norm: rows=%d cols=%d groups=%d dtype=%d", rows, cols, groups, dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(x && out, B2TTS_EINVAL, "gather_group_norm: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (gather_group_norm_kernel<T><<<rows, ROW_THREADS, 0, st>>>(x, rows_idx, static_cast<T*>(out), w, groups, eps, cols)));
  B2_CHECK_LAUNCH("gather_group_norm");
  return B2TTS_OK;
}

extern "C" int b2tts_xielu(void* y, const void* bias, const float* pq, int64_t rows, int cols, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(rows >= 0 && cols > 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "xielu: rows=%lld cols=%d dtype=%d", static_cast<long long>(rows), cols, dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(y && pq, B2TTS_EINVAL, "xielu: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t n = static_cast<size_t>(rows) * cols;
  LAT_DISPATCH(dtype, (xielu_kernel<T><<<flat_grid(n), 256, 0, st>>>(static_cast<T*>(y), static_cast<const T*>(bias), pq, n, cols)));
  B2_CHECK_LAUNCH("xielu");
  return B2TTS_OK;
}

extern "C" int b2tts_silu_mul(const void* gu, void* y, int64_t rows, int ff, int dtype, void* stream) {
  using namespace b2;
  using namespace b2::lat;
  B2_REQUIRE(rows >= 0 && ff > 0 && LAT_DTYPE_OK(dtype), B2TTS_EINVAL, "silu_mul: rows=%lld ff=%d dtype=%d", static_cast<long long>(rows), ff, dtype);
  if (rows == 0) return B2TTS_OK;
  B2_REQUIRE(gu && y, B2TTS_EINVAL, "silu_mul: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LAT_DISPATCH(dtype, (silu_mul_kernel<T><<<flat_grid(static_cast<size_t>(rows) * ff), 256, 0, st>>>(static_cast<const T*>(gu), static_cast<T*>(y),
                                                                                                  static_cast<size_t>(rows), ff)));
  B2_CHECK_LAUNCH("silu_mul");
  return B2TTS_OK;
}
