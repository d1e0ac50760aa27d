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
                           int H, int G, int d, int dv, int page, int window, float scale, int skip_single) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.z, g = blockIdx.y;
  const int len = seq_len[b];
  if (skip_single && len == 1) return;               // the streaming kernel below owns one-token rows
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
                                      int G, int d, int dv, int page, int window, float scale, int skip_single) {
  auto kern = window_sigmoid_attn_kernel<T, DVL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, WA_WARPS * 32, smem, st>>>(static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc),
                                          static_cast<T*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb, H, G, d,
                                          dv, page, window, scale, skip_single);
  return cudaSuccess;
}

// ------------------------------------------------------------------ one new token per sequence: stream the window once
// One CTA per (sequence, key/value head), 8 warps.  A key is read by LPK lanes, 16 bytes each, so a warp takes 32 / LPK
// keys per copy instruction.  The copies are asynchronous into a per-warp ring in shared memory (each lane owns its
// slots, so no barrier is needed), the pages of the window are looked up once per CTA, and so are the heads' distance
// terms.  The lane's slice of q stays in registers for every head of the group; a score is a dot over the slice plus
// log2(LPK) shuffles; the weighted values accumulate per lane and are summed over key groups and warps at the end, in
// a fixed order.  There is no split over keys: a window is a few hundred keys and the batch supplies the CTAs.
constexpr int WD_WARPS = 8;
constexpr int WD_UNROLL = 2;                      // key groups per ring stage
constexpr int WD_STAGES = 4;
constexpr size_t WD_RING_BYTES = static_cast<size_t>(WD_WARPS) * WD_STAGES * WD_UNROLL * 2 * 32 * 16;

template <typename T> struct WdVec;
template <> struct WdVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void cvt(const uint4& r, float* f) {
    f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y);
    f[4] = bf16lo(r.z); f[5] = bf16hi(r.z); f[6] = bf16lo(r.w); f[7] = bf16hi(r.w);
  }
};
template <> struct WdVec<float> {
  static constexpr int N = 4;
  __device__ static void cvt(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
};
template <typename T> __device__ __forceinline__ void wd_load(const T* p, float* f) {
  WdVec<T>::cvt(*reinterpret_cast<const uint4*>(p), f);
}

template <typename T, int LPK, int REP>
__global__ void __launch_bounds__(WD_WARPS * 32)
window_sigmoid_attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                  T* __restrict__ out, const int32_t* __restrict__ seq_start,
                                  const int32_t* __restrict__ seq_pos0, const int32_t* __restrict__ seq_len,
                                  const int32_t* __restrict__ block_tables, int bt_stride, const float* __restrict__ r1,
                                  const float* __restrict__ r2, const float* __restrict__ pb, int H, int G, int d, int dv,
                                  int page, int window, float scale, int use_tab) {
  constexpr int VEC = WdVec<T>::N;
  constexpr int KPI = 32 / LPK;                      // keys per warp load
  extern __shared__ __align__(16) unsigned char wd_smem[];
  uint4* ring = reinterpret_cast<uint4*>(wd_smem);   // [WD_WARPS][WD_STAGES][WD_UNROLL][K | V][32 lanes]
  float* red = reinterpret_cast<float*>(wd_smem + WD_RING_BYTES);                          // [WD_WARPS][rep][dv]
  const int b = blockIdx.z, g = blockIdx.y;
  const int len = seq_len[b];
  const int rep = H / G;
  const int n = seq_start[b];
  if (len <= 0) {                                    // padding row of a captured step: defined output
    for (int c = threadIdx.x; c < rep * dv; c += blockDim.x) out[static_cast<size_t>(n) * H * dv + g * rep * dv + c] = wa_from_f<T>(0.f);
    return;
  }
  if (len != 1) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / LPK, c0 = (lane % LPK) * VEC;
  const int p = seq_pos0[b];
  const int j_lo = max(0, p - window + 1);
  const int32_t* bt = block_tables + static_cast<size_t>(b) * bt_stride;
  const bool has_k = c0 < d, has_v = c0 < dv;
  float qv[REP][VEC], acc[REP][VEC], hr1[REP], hr2[REP], hpb[REP];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const bool ok = r < rep;
    const int h = g * rep + (ok ? r : 0);
    hr1[r] = r1[h]; hr2[r] = r2[h]; hpb[r] = pb[h];
#pragma unroll
    for (int i = 0; i < VEC; ++i) { qv[r][i] = 0.f; acc[r][i] = 0.f; }
    if (ok && has_k) wd_load(q + static_cast<size_t>(n) * H * d + h * d + c0, qv[r]);
  }
  // the window's pages, once: pages[i] = block table entry of page pg0 + i
  int32_t* pages = reinterpret_cast<int32_t*>(red + WD_WARPS * rep * dv);
  const int pg0 = j_lo / page;
  for (int i = threadIdx.x; i <= p / page - pg0; i += blockDim.x) pages[i] = bt[pg0 + i];
  // the heads' distance terms, once per CTA instead of once per lane and key:
  //   tab[r][dist] = log2(e) (r1 ln(1 + r2 dist) - pb),  weight = 1 / (1 + 2^(tab - log2(e) scale s))
  constexpr float LOG2E = 1.4426950408889634f;
  const int span = p - j_lo + 1;
  float* tab = reinterpret_cast<float*>(pages + (window + page - 1) / page + 2);
  if (use_tab)
    for (int i = threadIdx.x; i < rep * span; i += blockDim.x) {
      const int r = i / span, h = g * rep + r;
      tab[i] = LOG2E * (r1[h] * log1pf(r2[h] * static_cast<float>(i - r * span)) - pb[h]);
    }
  const float scale2 = scale * LOG2E;
  __syncthreads();
  // Each lane copies its own 16-byte slices of K and V asynchronously into its own slots of the warp's ring and reads
  // them back itself, so the ring needs no barrier: WD_STAGES - 1 stages are in flight while one is multiplied.
  uint4* myring = ring + static_cast<size_t>(warp) * WD_STAGES * WD_UNROLL * 2 * 32 + lane;
  const int step = WD_WARPS * KPI * WD_UNROLL;
  const int base0 = j_lo + warp * KPI * WD_UNROLL;
  const int n_it = base0 <= p ? (p - base0) / step + 1 : 0;
  auto issue = [&](int it) {
    uint4* st = myring + (it % WD_STAGES) * WD_UNROLL * 2 * 32;
#pragma unroll
    for (int u = 0; u < WD_UNROLL; ++u) {
      const int j = base0 + it * step + u * KPI + grp;
      const bool ok = j <= p;
      size_t slot = 0;
      if (ok) {
        const int pg = j / page;
        slot = static_cast<size_t>(pages[pg - pg0]) * page + (j - pg * page);
      }
      cp_async_16(st + (u * 2) * 32, k_cache + slot * G * d + g * d + (has_k ? c0 : 0), ok && has_k);
      cp_async_16(st + (u * 2 + 1) * 32, v_cache + slot * G * dv + g * dv + (has_v ? c0 : 0), ok && has_v);
    }
  };
#pragma unroll
  for (int s0 = 0; s0 < WD_STAGES - 1; ++s0) {
    if (s0 < n_it) issue(s0);
    cp_async_commit();
  }
  for (int it = 0; it < n_it; ++it) {
    cp_async_wait<WD_STAGES - 2>();                  // this thread's copies of stage `it` have landed
    if (it + WD_STAGES - 1 < n_it) issue(it + WD_STAGES - 1);
    cp_async_commit();
    const uint4* st = myring + (it % WD_STAGES) * WD_UNROLL * 2 * 32;
#pragma unroll
    for (int u = 0; u < WD_UNROLL; ++u) {
      const int j = base0 + it * step + u * KPI + grp;
      const float dist = static_cast<float>(p - j);
      float kf[VEC], vf[VEC];
      WdVec<T>::cvt(st[(u * 2) * 32], kf);
      WdVec<T>::cvt(st[(u * 2 + 1) * 32], vf);
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) s = fmaf(qv[r][i], kf[i], s);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        float w = 0.f;
        if (j <= p && r < rep) {
          if (use_tab) {
            w = __fdividef(1.0f, 1.0f + exp2f(tab[r * span + (p - j)] - s * scale2));
          } else {
            const float z = s * scale - hr1[r] * log1pf(hr2[r] * dist) + hpb[r];
            w = 1.0f / (1.0f + expf(-z));
          }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[r][i] = fmaf(w, vf[i], acc[r][i]);
      }
    }
  }
  cp_async_wait<0>();
  // over the key groups of the warp, then over the warps
#pragma unroll
  for (int r = 0; r < REP; ++r)
#pragma unroll
    for (int i = 0; i < VEC; ++i)
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], o);
  if (grp == 0 && has_v) {
#pragma unroll
    for (int r = 0; r < REP; ++r)
      if (r < rep)
#pragma unroll
        for (int i = 0; i < VEC; ++i) red[(warp * rep + r) * dv + c0 + i] = acc[r][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rep * dv; idx += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WD_WARPS; ++w) t += red[w * rep * dv + idx];
    out[static_cast<size_t>(n) * H * dv + g * rep * dv + idx] = wa_from_f<T>(t);
  }
}

template <typename T, int LPK, int REP>
static cudaError_t launch_window_decode(dim3 grid, size_t smem, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                        const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* bt,
                                        int bt_stride, const float* r1, const float* r2, const float* pb, int H, int G, int d, int dv,
                                        int page, int window, float scale, int use_tab) {
  auto kern = window_sigmoid_attn_decode_kernel<T, LPK, REP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, WD_WARPS * 32, smem, st>>>(static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc),
                                          static_cast<T*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb, H, G, d, dv,
                                          page, window, scale, use_tab);
  return cudaSuccess;
}

// ------------------------------------------------------------------ prompt portions on the tensor cores (bf16)
// 64 query tokens of a head per CTA (4 warps x 16 rows), key tiles gathered through the block table into padded
// shared-memory rows.  S = Q K^T and O += P V run as m16n8k16 bf16 MMAs with float accumulators held in registers; the
// weights are computed in float from the float scores, and enter the second product as a bf16 pair hi + lo
// (lo = bf16(w - hi)), i.e. with 16 mantissa bits, so that no weight is rounded to bf16.  The distance bias of the
// head, r1 * ln(1 + r2 * dist) - pb for dist < window, is tabulated once per CTA.

// 2^x and 1/x on the special-function unit (about 2 ulp; denormal results flush to zero, 2^big = inf, 1/inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x, y);                              // one rounding instruction for the pair
  lo = pack_bf16(x - bf16lo(hi), y - bf16hi(hi));
}

constexpr int WM_BM = 64, WM_BN = 64;

// REPB query heads of one key/value group share the CTA (4 warps each) and with it every K/V tile of BN keys; the tiles
// arrive by 16-byte asynchronous copies into a two-stage ring, so tile t + 1 is in flight while tile t is multiplied.
// Tiles that lie wholly inside the window of all 16 rows of a warp take a path without per-element tests.
template <int D, int DV, int REPB, int BN>
__global__ void __launch_bounds__(128 * REPB, 4 / REPB)
window_sigmoid_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                               const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                               const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                               const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_tables, int bt_stride,
                               const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb,
                               int H, int G, int page, int page_shift, int window, float scale) {
  static_assert(D == DV, "one slot computation serves the K and the V chunk");
  constexpr int WM_BN = BN;                          // keys per tile
  constexpr int QS = D + 8, VS = DV + 8;             // padded rows: 16-byte aligned, ldmatrix rows land in distinct banks
  constexpr int NT = 128 * REPB;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char wm_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(wm_smem);       // [REPB][BM][QS]
  __nv_bfloat16* Ks = Qs + REPB * WM_BM * QS;                          // [2][BN][QS]
  __nv_bfloat16* Vs = Ks + 2 * WM_BN * QS;                             // [2][BN][VS]
  float* tab = reinterpret_cast<float*>(Vs + 2 * WM_BN * VS);          // [REPB][window]
  const int b = blockIdx.z, h0 = blockIdx.y * REPB, g = h0 / (H / G);
  const int len = seq_len[b];
  const int t0 = blockIdx.x * WM_BM;
  if (len <= 1 || t0 >= len) return;                 // one-token and padding rows belong to the streaming kernel
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hw = warp >> 2, wr = warp & 3;           // this warp: head h0 + hw, rows wr * 16 ..
  const int start = seq_start[b], pos0 = seq_pos0[b];
  const int32_t* bt = block_tables + static_cast<size_t>(b) * bt_stride;
  for (int idx = tid; idx < REPB * WM_BM * (D / 8); idx += NT) {
    const int hr = idx / (WM_BM * (D / 8)), r = idx / (D / 8) % WM_BM, ch = idx % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + r < len) v = ldg_v4(q + static_cast<size_t>(start + t0 + r) * H * D + (h0 + hr) * D + ch * 8);
    *reinterpret_cast<uint4*>(Qs + (hr * WM_BM + r) * QS + ch * 8) = v;
  }
  // log2(e) * (r1 ln(1 + r2 dist) - pb): the weight is 1 / (1 + 2^(tab[dist] - log2(e) scale s))
  for (int i = tid; i < REPB * window; i += NT) {
    const int h = h0 + i / window, dist = i % window;
    tab[i] = LOG2E * (r1[h] * log1pf(r2[h] * static_cast<float>(dist)) - pb[h]);
  }
  const float scale2 = scale * LOG2E;
  const int t_hi = min(len - 1, t0 + WM_BM - 1);
  const int j_lo = max(0, pos0 + t0 - window + 1), j_hi = pos0 + t_hi;
  const int row_lo = wr * 16 + (lane >> 2);
  const int p_lo = pos0 + t0 + row_lo, p_hi = p_lo + 8;
  const bool ok_lo = t0 + row_lo < len, ok_hi = t0 + row_lo + 8 < len;
  const float* mytab = tab + hw * window;
  float oacc[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;

  // four threads per key: one slot computation, then the thread's chunks lch, lch + 4, ... of the key's K and V rows
  static_assert(NT / 4 == WM_BN && (D / 8) % 4 == 0, "loader: 4 threads per key");
  const int lkey = tid >> 2, lch = tid & 3;
  auto load_tile = [&](int stage, int j0) {
    const int j = j0 + lkey;
    const bool ok = j <= j_hi;
    size_t slot = 0;
    if (ok) {
      const int pg = page_shift >= 0 ? j >> page_shift : j / page;
      slot = static_cast<size_t>(bt[pg]) * page + (j - pg * page);
    }
    const __nv_bfloat16* ksrc = k_cache + (slot * G + g) * D + lch * 8;
    const __nv_bfloat16* vsrc = v_cache + (slot * G + g) * DV + lch * 8;
    __nv_bfloat16* kd = Ks + (stage * WM_BN + lkey) * QS + lch * 8;
    __nv_bfloat16* vd = Vs + (stage * WM_BN + lkey) * VS + lch * 8;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      cp_async_16(kd + i * 32, ksrc + i * 32, ok);
      cp_async_16(vd + i * 32, vsrc + i * 32, ok);
    }
  };
  const int n_tiles = (j_hi - j_lo) / WM_BN + 1;
  load_tile(0, j_lo);
  cp_async_commit();
  for (int t = 0; t < n_tiles; ++t) {
    const int j0 = j_lo + t * WM_BN;
    cp_async_wait<0>();
    __syncthreads();                                 // tile t has landed (Q and the table too); tile t - 1 is consumed
    if (t + 1 < n_tiles) load_tile((t + 1) & 1, j0 + WM_BN);
    cp_async_commit();
    const __nv_bfloat16* Kt = Ks + (t & 1) * WM_BN * QS;
    const __nv_bfloat16* Vt = Vs + (t & 1) * WM_BN * VS;
    // this warp's rows see keys p - window + 1 .. p: skip a tile none of its 16 rows can see
    const int wp_lo = pos0 + t0 + wr * 16, wp_hi = wp_lo + 15;
    if (j0 > wp_hi || j0 + WM_BN - 1 < wp_lo - window + 1 || t0 + wr * 16 >= len) continue;
    float sacc[WM_BN / 8][4];
#pragma unroll
    for (int i = 0; i < WM_BN / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], Qs + (hw * WM_BM + wr * 16 + (lane & 15)) * QS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < WM_BN / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, Kt + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * QS + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(sacc[2 * np], a, b0, b1);
        mma_bf16_16816(sacc[2 * np + 1], a, b2, b3);
      }
    }
    // a tile wholly inside every row's window needs no per-element test: the distance is a compile-time offset from
    // the lane's first one, and a weight is one fused multiply-add, ex2, add and reciprocal
    const bool inner = j0 + WM_BN - 1 <= wp_lo && j0 >= wp_hi - window + 1 && t0 + wr * 16 + 15 < len;
    if (inner) {
      const float* tl = mytab + (p_lo - j0 - 2 * (lane & 3));
      const float* th = tl + 8;
#pragma unroll
      for (int nt = 0; nt < WM_BN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float bias = (e < 2 ? tl : th)[-(nt * 8 + (e & 1))];
          sacc[nt][e] = rcp_approx(1.0f + ex2_approx(fmaf(-scale2, sacc[nt][e], bias)));
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < WM_BN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + nt * 8 + 2 * (lane & 3) + (e & 1);
          const int dist = (e < 2 ? p_lo : p_hi) - j;
          const bool ok = (e < 2 ? ok_lo : ok_hi) && dist >= 0 && dist < window;
          float w = 0.f;
          if (ok) w = rcp_approx(1.0f + ex2_approx(fmaf(-scale2, sacc[nt][e], mytab[dist])));
          sacc[nt][e] = w;
        }
      }
    }
#pragma unroll
    for (int kk = 0; kk < WM_BN / 16; ++kk) {
      uint32_t ah[4], al[4];
      split_bf16(sacc[2 * kk][0], sacc[2 * kk][1], ah[0], al[0]);
      split_bf16(sacc[2 * kk][2], sacc[2 * kk][3], ah[1], al[1]);
      split_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], ah[2], al[2]);
      split_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
      for (int np = 0; np < DV / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, Vt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VS + np * 16 + (lane >> 4) * 8);
        mma_bf16_16816(oacc[2 * np], ah, b0, b1);
        mma_bf16_16816(oacc[2 * np], al, b0, b1);
        mma_bf16_16816(oacc[2 * np + 1], ah, b2, b3);
        mma_bf16_16816(oacc[2 * np + 1], al, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!(half ? ok_hi : ok_lo)) continue;
    __nv_bfloat16* o = out + static_cast<size_t>(start + t0 + row_lo + 8 * half) * H * DV + (h0 + hw) * DV + 2 * (lane & 3);
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt)
      *reinterpret_cast<uint32_t*>(o + nt * 8) = pack_bf16(oacc[nt][2 * half], oacc[nt][2 * half + 1]);
  }
}

template <int D, int REPB, int BN>
static cudaError_t launch_window_mma(int max_new, int n_seqs, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                     const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* bt,
                                     int bt_stride, const float* r1, const float* r2, const float* pb, int H, int G, int page,
                                     int window, float scale) {
  auto kern = window_sigmoid_attn_mma_kernel<D, D, REPB, BN>;
  const size_t smem = sizeof(__nv_bfloat16) * (REPB * WM_BM + 4 * BN) * (D + 8) + sizeof(float) * REPB * window;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  using B = __nv_bfloat16;
  int page_shift = -1;
  if ((page & (page - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page; ++page_shift) {}
  const dim3 grid((max_new + WM_BM - 1) / WM_BM, H / REPB, n_seqs);
  kern<<<grid, 128 * REPB, smem, st>>>(static_cast<const B*>(q), static_cast<const B*>(kc), static_cast<const B*>(vc),
                                       static_cast<B*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb, H, G, page,
                                       page_shift, window, scale);
  return cudaSuccess;
}

// ------------------------------------------------------------------ one new token per sequence on the tensor cores (bf16)
// The rows of the m16n8k16 tile are the query HEADS of one key/value group (rep <= 16, the rest zero), so one pass over
// K and V serves the whole group with a handful of instructions per key: S = Q K^T for 16 keys is D / 8 MMAs, the
// weights are computed once per (head, key) from the float scores and the per-CTA distance table, and O += P V takes
// D / 4 MMAs with the weights as a bf16 pair hi + lo.  One CTA per (sequence, key/value head), 4 warps; warp w owns the
// 16-key tiles w, w + 4, ... of the window and streams them through its own two-stage ring of 16-byte asynchronous
// copies (no CTA barrier in the loop); the warps' partial outputs are added in a fixed order at the end.
constexpr int WT_WARPS = 4, WT_KEYS = 16;

template <int D>
__global__ void __launch_bounds__(WT_WARPS * 32)
window_sigmoid_attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                                      const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                                      const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_pos0,
                                      const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_tables, int bt_stride,
                                      const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb,
                                      int H, int G, int page, int window, float scale) {
  constexpr int RS = D + 8, CH = D / 8;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char wt_smem[];
  const int b = blockIdx.z, g = blockIdx.y;
  const int len = seq_len[b];
  const int rep = H / G;
  const int n = seq_start[b];
  if (len <= 0) {                                    // padding row of a captured step: defined output
    for (int c = threadIdx.x; c < rep * D; c += blockDim.x) out[static_cast<size_t>(n) * H * D + g * rep * D + c] = __float2bfloat16_rn(0.f);
    return;
  }
  if (len != 1) return;
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(wt_smem);    // [WARPS][2 stages][K | V][KEYS][RS]
  __nv_bfloat16* Qs = ring + WT_WARPS * 2 * 2 * WT_KEYS * RS;         // [16][RS]
  float* red = reinterpret_cast<float*>(Qs + 16 * RS);                // [WARPS][rep][D]
  int32_t* pages = reinterpret_cast<int32_t*>(red + WT_WARPS * rep * D);
  float* tab = reinterpret_cast<float*>(pages + (window + page - 1) / page + 2);   // [rep][span]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = seq_pos0[b];
  const int j_lo = max(0, p - window + 1), span = p - j_lo + 1;
  const int32_t* bt = block_tables + static_cast<size_t>(b) * bt_stride;
  for (int idx = tid; idx < 16 * CH; idx += blockDim.x) {
    const int r = idx / CH, ch = idx % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rep) v = ldg_v4(q + static_cast<size_t>(n) * H * D + (g * rep + r) * D + ch * 8);
    *reinterpret_cast<uint4*>(Qs + r * RS + ch * 8) = v;
  }
  const int pg0 = j_lo / page;
  for (int i = tid; i <= p / page - pg0; i += blockDim.x) pages[i] = bt[pg0 + i];
  for (int i = tid; i < rep * span; i += blockDim.x) {
    const int r = i / span, h = g * rep + r;
    tab[i] = LOG2E * (r1[h] * log1pf(r2[h] * static_cast<float>(i - r * span)) - pb[h]);
  }
  const float scale2 = scale * LOG2E;
  __syncthreads();
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldsm_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], Qs + (lane & 15) * RS + ks * 16 + (lane >> 4) * 8);
  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
  __nv_bfloat16* myring = ring + warp * 2 * 2 * WT_KEYS * RS;
  const int n_tiles = (span + WT_KEYS - 1) / WT_KEYS;
  const int n_my = warp < n_tiles ? (n_tiles - 1 - warp) / WT_WARPS + 1 : 0;
  auto issue = [&](int i) {
    const int j0 = j_lo + (warp + i * WT_WARPS) * WT_KEYS;
    __nv_bfloat16* kd = myring + (i & 1) * 2 * WT_KEYS * RS;
    __nv_bfloat16* vd = kd + WT_KEYS * RS;
    const int jk = j0 + (lane & 15);                 // lanes 0..15 (and their mirrors) look one key's slot up each
    int slot_k = 0;
    if (jk <= p) {
      const int pg = jk / page;
      slot_k = pages[pg - pg0] * page + (jk - pg * page);
    }
#pragma unroll
    for (int c = lane; c < WT_KEYS * CH; c += 32) {
      const int key = c / CH, ch = c % CH;
      const size_t slot = static_cast<size_t>(__shfl_sync(0xffffffffu, slot_k, key));
      const bool ok = j0 + key <= p;
      cp_async_16(kd + key * RS + ch * 8, k_cache + (slot * G + g) * D + ch * 8, ok);
      cp_async_16(vd + key * RS + ch * 8, v_cache + (slot * G + g) * D + ch * 8, ok);
    }
  };
  if (n_my > 0) issue(0);
  cp_async_commit();
  for (int i = 0; i < n_my; ++i) {
    if (i + 1 < n_my) issue(i + 1);
    cp_async_commit();
    cp_async_wait<1>();                              // this lane's copies of tile i have landed ...
    __syncwarp();                                    // ... and so have the other lanes'
    const int j0 = j_lo + (warp + i * WT_WARPS) * WT_KEYS;
    const __nv_bfloat16* Kt = myring + (i & 1) * 2 * WT_KEYS * RS;
    const __nv_bfloat16* Vt = Kt + WT_KEYS * RS;
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(b0, b1, b2, b3, Kt + ((lane >> 4) * 8 + (lane & 7)) * RS + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16_16816(sacc[0], qa[ks], b0, b1);
      mma_bf16_16816(sacc[1], qa[ks], b2, b3);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (lane >> 2) + (e >= 2 ? 8 : 0);
        const int j = j0 + nt * 8 + 2 * (lane & 3) + (e & 1);
        float w = 0.f;
        if (row < rep && j <= p) w = __fdividef(1.0f, 1.0f + exp2f(tab[row * span + (p - j)] - sacc[nt][e] * scale2));
        sacc[nt][e] = w;
      }
    uint32_t ah[4], al[4];
    split_bf16(sacc[0][0], sacc[0][1], ah[0], al[0]);
    split_bf16(sacc[0][2], sacc[0][3], ah[1], al[1]);
    split_bf16(sacc[1][0], sacc[1][1], ah[2], al[2]);
    split_bf16(sacc[1][2], sacc[1][3], ah[3], al[3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(b0, b1, b2, b3, Vt + (((lane >> 3) & 1) * 8 + (lane & 7)) * RS + np * 16 + (lane >> 4) * 8);
      mma_bf16_16816(oacc[2 * np], ah, b0, b1);
      mma_bf16_16816(oacc[2 * np], al, b0, b1);
      mma_bf16_16816(oacc[2 * np + 1], ah, b2, b3);
      mma_bf16_16816(oacc[2 * np + 1], al, b2, b3);
    }
    __syncwarp();                                    // every lane is done with this stage before it is refilled
  }
  cp_async_wait<0>();
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * (lane & 3);
    const int ra = lane >> 2, rb = ra + 8;
    if (ra < rep) { red[(warp * rep + ra) * D + col] = oacc[nt][0]; red[(warp * rep + ra) * D + col + 1] = oacc[nt][1]; }
    if (rb < rep) { red[(warp * rep + rb) * D + col] = oacc[nt][2]; red[(warp * rep + rb) * D + col + 1] = oacc[nt][3]; }
  }
  __syncthreads();
  for (int idx = tid; idx < rep * D; idx += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WT_WARPS; ++w) t += red[w * rep * D + idx];
    out[static_cast<size_t>(n) * H * D + g * rep * D + idx] = __float2bfloat16_rn(t);
  }
}

template <int D>
static size_t window_decode_mma_smem(int rep, int page, int window) {
  return sizeof(__nv_bfloat16) * (WT_WARPS * 2 * 2 * WT_KEYS + 16) * (D + 8) + sizeof(float) * WT_WARPS * rep * D +
         sizeof(int32_t) * ((window + page - 1) / page + 2) + sizeof(float) * rep * window;
}

template <int D>
static cudaError_t launch_window_decode_mma(int n_seqs, cudaStream_t st, const void* q, const void* kc, const void* vc, void* out,
                                            const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                            const int32_t* bt, int bt_stride, const float* r1, const float* r2, const float* pb, int H,
                                            int G, int page, int window, float scale) {
  auto kern = window_sigmoid_attn_decode_mma_kernel<D>;
  const size_t smem = window_decode_mma_smem<D>(H / G, page, window);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  using B = __nv_bfloat16;
  kern<<<dim3(1, G, n_seqs), WT_WARPS * 32, smem, st>>>(static_cast<const B*>(q), static_cast<const B*>(kc), static_cast<const B*>(vc),
                                                        static_cast<B*>(out), seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb,
                                                        H, G, page, window, scale);
  return cudaSuccess;
}

template <typename T, int LPK>
static cudaError_t launch_window_decode_rep(int rep, dim3 grid, size_t smem, cudaStream_t st, const void* q, const void* kc, const void* vc,
                                            void* out, const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                            const int32_t* bt, int bt_stride, const float* r1, const float* r2, const float* pb, int H,
                                            int G, int d, int dv, int page, int window, float scale, int use_tab) {
#define WD_GO(R) launch_window_decode<T, LPK, R>(grid, smem, st, q, kc, vc, out, seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, pb, \
                                                 H, G, d, dv, page, window, scale, use_tab)
  if (rep <= 1) return WD_GO(1);
  if (rep <= 2) return WD_GO(2);
  if (rep <= 4) return WD_GO(4);
  return WD_GO(8);
#undef WD_GO
}

template <typename T>
static cudaError_t launch_window_decode_any(int lpk, int rep, dim3 grid, size_t smem, cudaStream_t st, const void* q, const void* kc,
                                            const void* vc, void* out, const int32_t* seq_start, const int32_t* seq_pos0,
                                            const int32_t* seq_len, const int32_t* bt, int bt_stride, const float* r1, const float* r2,
                                            const float* pb, int H, int G, int d, int dv, int page, int window, float scale,
                                            int use_tab) {
#define WD_GO(L) launch_window_decode_rep<T, L>(rep, grid, smem, st, q, kc, vc, out, seq_start, seq_pos0, seq_len, bt, bt_stride, r1, r2, \
                                                pb, H, G, d, dv, page, window, scale, use_tab)
  if (lpk <= 8) return WD_GO(8);
  if (lpk <= 16) return WD_GO(16);
  return WD_GO(32);
#undef WD_GO
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  // one-token rows: the streaming kernel, when the head sizes allow 16-byte slices and the group fits its registers
  const int vec = dtype == B2TTS_DTYPE_BF16 ? 8 : 4;
  const int widest = dim > vdim ? dim : vdim;
  const bool stream_ok = dim % vec == 0 && vdim % vec == 0 && widest <= 32 * vec && rep <= 8 && aligned16(q) && aligned16(k_cache) &&
                         aligned16(v_cache);
  const bool tensor_shape = stream_ok && dtype == B2TTS_DTYPE_BF16 && dim == vdim && (dim == 32 || dim == 64 || dim == 96 || dim == 128);
  size_t smem_t = 0;
  if (tensor_shape && rep <= 16)
    smem_t = dim == 32 ? window_decode_mma_smem<32>(rep, page, window) : dim == 64 ? window_decode_mma_smem<64>(rep, page, window)
           : dim == 96 ? window_decode_mma_smem<96>(rep, page, window) : window_decode_mma_smem<128>(rep, page, window);
  const bool decode_tensor = smem_t > 0 && smem_t <= 200 * 1024;
  if (decode_tensor) {
#define WT_GO(DD) e = launch_window_decode_mma<DD>(n_seqs, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len, block_tables, \
                                                   bt_stride, r1, r2, pb, heads, kv_heads, page, window, scale)
    if (dim == 32) WT_GO(32); else if (dim == 64) WT_GO(64); else if (dim == 96) WT_GO(96); else WT_GO(128);
#undef WT_GO
    if (e != cudaSuccess) return cuda_fail(e, "window_sigmoid_attn (one token, tensor)");
    B2_CHECK_LAUNCH("window_sigmoid_attn (one token, tensor)");
    if (max_new == 1) return B2TTS_OK;
  } else if (stream_ok) {
    const int lpk = (widest + vec - 1) / vec;
    const size_t tab_bytes = sizeof(float) * rep * window;
    const int use_tab = tab_bytes <= 64 * 1024;          // larger windows compute the distance term per key
    const size_t smem_d = WD_RING_BYTES + sizeof(float) * WD_WARPS * rep * vdim + sizeof(int32_t) * ((window + page - 1) / page + 2) +
                          (use_tab ? tab_bytes : 0);
    const dim3 grid_d(1, kv_heads, n_seqs);
    if (dtype == B2TTS_DTYPE_BF16)
      e = launch_window_decode_any<__nv_bfloat16>(lpk, rep, grid_d, smem_d, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len,
                                                  block_tables, bt_stride, r1, r2, pb, heads, kv_heads, dim, vdim, page, window, scale, use_tab);
    else
      e = launch_window_decode_any<float>(lpk, rep, grid_d, smem_d, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len,
                                          block_tables, bt_stride, r1, r2, pb, heads, kv_heads, dim, vdim, page, window, scale, use_tab);
    if (e != cudaSuccess) return cuda_fail(e, "window_sigmoid_attn (streaming)");
    B2_CHECK_LAUNCH("window_sigmoid_attn (streaming)");
    if (max_new == 1) return B2TTS_OK;
  }
  // prompt portions in bf16 with a supported head size: the tensor-core kernel
  if (stream_ok && dtype == B2TTS_DTYPE_BF16 && dim == vdim && (dim == 32 || dim == 64 || dim == 96 || dim == 128) && window <= 8192) {
    // One head and 32-key tiles per CTA, four CTAs per SM: independent CTAs overlap their MMA and weight phases better
    // than a wider CTA in which two heads share the K/V tiles (306 against 322 us at 4 x 2048 tokens, window 1024).
#define WM_GO(DD) e = launch_window_mma<DD, 1, 32>(max_new, n_seqs, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len, \
                                                   block_tables, bt_stride, r1, r2, pb, heads, kv_heads, page, window, scale)
    if (dim == 32) WM_GO(32); else if (dim == 64) WM_GO(64); else if (dim == 96) WM_GO(96); else WM_GO(128);
#undef WM_GO
    if (e != cudaSuccess) return cuda_fail(e, "window_sigmoid_attn (tensor)");
    B2_CHECK_LAUNCH("window_sigmoid_attn (tensor)");
    return B2TTS_OK;
  }
  const int skip_single = stream_ok ? 1 : 0;
  const int d4 = (dim + 3) & ~3;
  const size_t smem = sizeof(float) * (static_cast<size_t>(WA_ROWS) * d4 + WA_BK * (d4 + 4) + static_cast<size_t>(WA_BK) * vdim +
                                       WA_ROWS * (WA_BK + 1));
  B2_REQUIRE(smem <= 200 * 1024, B2TTS_EUNSUPPORTED, "window_sigmoid_attn: head size %d needs %zu bytes of shared memory", dim, smem);
  const dim3 grid((static_cast<unsigned>(max_new) * rep + WA_ROWS - 1) / WA_ROWS, kv_heads, n_seqs);
  const int dvl = (vdim + 31) / 32;
#define WA_GO(T, L) e = launch_window_attn<T, L>(grid, smem, st, q, k_cache, v_cache, out, seq_start, seq_pos0, seq_len, block_tables, \
                                                 bt_stride, r1, r2, pb, heads, kv_heads, dim, vdim, page, window, scale, skip_single)
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
