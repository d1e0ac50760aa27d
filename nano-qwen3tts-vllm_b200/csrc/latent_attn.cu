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


// ------------------------------------------------------------------ tensor-core kernel (bf16)
// A CTA owns 16 query rows: G consecutive tokens of one sequence times up to 16 heads (G = 16 / heads when a sequence
// has fewer than 16 heads; a decoded token is a tile with one token).  All rows read the SAME cached rows, so a tile of
// 64 keys is staged once in shared memory ([key][c | kr], two stages filled by 16-byte asynchronous copies through the
// block table) and used twice: as the key operand of S = Q K^T (each warp scores its own 8 or 16 keys over the whole
// row width) and, its first r columns read transposed, as the value operand of O += P V (each warp owns r / NW
// columns of O in registers).  Between the two products the 16 x 64 scores cross shared memory as floats, where the
// running maximum, the sum and the weights are formed in float (the sink starts the maximum and the sum).
constexpr int LM_KT = 64;                       // keys per tile

__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}

struct LatentMmaSmem {
  int q_off, k_off, s_off, p_off, st_off, total, ldk;   // byte offsets; ldk = padded row length in elements
};
static LatentMmaSmem latent_mma_smem(int r, int dr) {
  LatentMmaSmem m;
  const int dkp = (r + dr + 15) / 16 * 16;
  m.ldk = dkp + 8;
  m.q_off = 0;
  m.k_off = 16 * m.ldk * 2;
  m.s_off = m.k_off + 2 * LM_KT * m.ldk * 2;
  m.p_off = m.s_off + 16 * LM_KT * 4;
  m.st_off = m.p_off + 16 * (LM_KT + 8) * 2;
  m.total = m.st_off + 16 * 4 * 4;
  return m;
}

template <int NW, int NT>
__global__ void __launch_bounds__(NW * 32)
latent_attn_mma_kernel(const LatentAttnArgs a, const LatentMmaSmem sm) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.q_off);
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.k_off);
  float* ss = reinterpret_cast<float*>(smem_raw + sm.s_off);
  __nv_bfloat16* ps = reinterpret_cast<__nv_bfloat16*>(smem_raw + sm.p_off);
  float* row_m = reinterpret_cast<float*>(smem_raw + sm.st_off);
  float* row_l = row_m + 16;
  float* row_alpha = row_l + 16;
  int* row_pos = reinterpret_cast<int*>(row_alpha + 16);
  constexpr int THREADS = NW * 32, LDP = LM_KT + 8, SN = LM_KT / 8 / NW;      // SN: score n-tiles per warp
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ldk = sm.ldk, dkp = ldk - 8, Dk = a.r + a.dr;
  const int b = blockIdx.y;
  const int len = a.seq_len[b];
  const int hpc = min(a.H, 16), hblocks = (a.H + 15) / 16, G = 16 / hpc;
  const int tile = blockIdx.x / hblocks, hb = blockIdx.x % hblocks;
  const int tl0 = tile * G;
  if (tl0 >= len) return;
  const int pos0 = a.seq_pos0[b], start = a.seq_start[b];
  const int n_tok = min(G, len - tl0);
  const int pos_first = pos0 + tl0, pos_last = pos_first + n_tok - 1;
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(a.cache);
  const int32_t* bt = a.block_tables + b * a.bt_stride;
  const int j_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int n_tiles = (pos_last - j_lo) / LM_KT + 1;

  // a warp copies whole rows: the page lookup is once per key and uniform over the warp, the lanes stride over the
  // row's 16-byte chunks; keys past the last query and the padding chunk are zero-filled
  auto load_tile = [&](int t, int stage) {
    __nv_bfloat16* dst = ks + static_cast<size_t>(stage) * LM_KT * ldk;
    const int cpr = dkp / 8, real = Dk / 8;
    // lane i looks up the i-th key of this warp: all the table reads of a tile are in flight together
    long long my = -1;
    if (lane < LM_KT / NW) {
      const int j = j_lo + t * LM_KT + warp + lane * NW;
      if (j <= pos_last) my = (static_cast<long long>(bt[j / a.page]) * a.page + j % a.page) * Dk;
    }
#pragma unroll
    for (int i = 0; i < LM_KT / NW; ++i) {
      const long long off = __shfl_sync(0xffffffffu, my, i);
      const bool in = off >= 0;
      const __nv_bfloat16* src = cache + (in ? off : 0);
      __nv_bfloat16* drow = dst + (warp + i * NW) * ldk;
      for (int ch = lane; ch < cpr; ch += 32) cp_async_16(drow + ch * 8, src + ch * 8, in && ch < real);
    }
    cp_async_commit();
  };
  load_tile(0, 0);

  // ---- the 16 query rows: [ql | rotate(qr)] as bf16, zero rows where the tile has no token or head
  if (tid < 16) {
    const int tl = tid / hpc, h = hb * 16 + tid % hpc;
    const bool ok = tl < n_tok && h < a.H;
    row_pos[tid] = ok ? pos_first + tl : -1;
    row_m[tid] = ok ? a.sink[h] : 0.f;
    row_l[tid] = 1.0f;
  }
  for (int row = warp; row < 16; row += NW) {
    const int tl = row / hpc, h = hb * 16 + row % hpc;
    const bool ok = tl < n_tok && h < a.H;
    const int tok = start + tl0 + tl;
    const __nv_bfloat16* ql = static_cast<const __nv_bfloat16*>(a.ql) + tok * a.ql_tok + h * a.ql_head;
    const __nv_bfloat16* qr = static_cast<const __nv_bfloat16*>(a.qr) + tok * a.qr_tok + h * a.qr_head;
    for (int c0 = lane * 2; c0 < dkp; c0 += 64) {
      float v0 = 0.f, v1 = 0.f;
      if (ok && c0 < a.r) {
        v0 = __bfloat162float(ql[c0]);
        v1 = __bfloat162float(ql[c0 + 1]);
      } else if (ok && c0 < Dk) {
        const int d = c0 - a.r;
        const float u = __bfloat162float(qr[d]), w = __bfloat162float(qr[d + 1]);
        if (d + 1 < a.rot_dims) {
          float sn, cs;
          sincosf(static_cast<float>(pos_first + tl) * a.freq[d / 2], &sn, &cs);
          sn *= a.rot_mult; cs *= a.rot_mult;
          v0 = u * cs - w * sn;
          v1 = w * cs + u * sn;
        } else { v0 = u; v1 = w; }
      }
      *reinterpret_cast<__nv_bfloat162*>(qs + row * ldk + c0) = __floats2bfloat162_rn(v0, v1);
    }
  }

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  const int col0 = warp * NT * 8;                                   // this warp's columns of O

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < n_tiles) { load_tile(t + 1, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const __nv_bfloat16* kt = ks + static_cast<size_t>(stage) * LM_KT * ldk;
    // ---- S = Q K^T for this warp's keys
    float sc[SN][2][4];                          // two accumulators per n-tile: alternate k-steps do not wait on each other
#pragma unroll
    for (int i = 0; i < SN; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[i][0][e] = sc[i][1][e] = 0.f;
    const __nv_bfloat16* q_lane = qs + (lane & 15) * ldk + (lane >> 4) * 8;
    const __nv_bfloat16* k_lane = kt + (warp * SN * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < dkp; k0 += 64) {       // the loads of four k-steps are issued before their products
      uint32_t af[4][4], bf[4][SN][2];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + 16 * u;
        if (k < dkp) {
          ldsm_x4(af[u][0], af[u][1], af[u][2], af[u][3], q_lane + k);
#pragma unroll
          for (int i = 0; i < SN; ++i) ldsm_x2(bf[u][i][0], bf[u][i][1], k_lane + i * 8 * ldk + k);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (k0 + 16 * u < dkp) {
#pragma unroll
          for (int i = 0; i < SN; ++i) mma_bf16_16816(sc[i][u & 1], af[u], bf[u][i][0], bf[u][i][1]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < SN; ++i) {
      const int n0 = (warp * SN + i) * 8 + (lane & 3) * 2, r0 = lane >> 2;
      ss[r0 * LM_KT + n0] = sc[i][0][0] + sc[i][1][0];
      ss[r0 * LM_KT + n0 + 1] = sc[i][0][1] + sc[i][1][1];
      ss[(r0 + 8) * LM_KT + n0] = sc[i][0][2] + sc[i][1][2];
      ss[(r0 + 8) * LM_KT + n0 + 1] = sc[i][0][3] + sc[i][1][3];
    }
    __syncthreads();
    // ---- running maximum, sum and weights, in float; a warp takes rows warp, warp + NW, ..
    for (int r2 = 2 * warp; r2 < 16; r2 += 2 * NW) {       // half a warp per row, four keys per lane
      const int row = r2 + (lane >> 4), l16 = lane & 15;
      const int rp = row_pos[row];
      float sv[4];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk = l16 + 16 * e;
        const int j = j_lo + t * LM_KT + kk;
        const bool vis = j <= rp && (a.window == 0 || rp - j < a.window);
        sv[e] = vis ? ss[row * LM_KT + kk] * a.scale : -INFINITY;
        mx = fmaxf(mx, sv[e]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = row_m[row];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pe = expf(sv[e] - m_new);                                  // exp(-inf) = 0 for hidden keys
        sum += pe;
        ps[row * LDP + l16 + 16 * e] = __float2bfloat16_rn(pe);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncwarp();
      if (l16 == 0) {
        const float alpha = expf(m_old - m_new);
        row_m[row] = m_new;
        row_l[row] = row_l[row] * alpha + sum;
        row_alpha[row] = alpha;
      }
    }
    __syncthreads();
    // ---- O = O * alpha + P V, V = the first r columns of the key tile
    {
      const float a0 = row_alpha[lane >> 2], a1 = row_alpha[(lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) { acc[i][0] *= a0; acc[i][1] *= a0; acc[i][2] *= a1; acc[i][3] *= a1; }
#pragma unroll
      for (int kk = 0; kk < LM_KT; kk += 16) {
        uint32_t pf[4];
        ldsm_x4(pf[0], pf[1], pf[2], pf[3], ps + (lane & 15) * LDP + kk + (lane >> 4) * 8);
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          uint32_t b0, b1;
          ldsm_x2_t(b0, b1, kt + (kk + (lane & 15)) * ldk + col0 + i * 8);
          mma_bf16_16816(acc[i], pf, b0, b1);
        }
      }
    }
    __syncthreads();
  }
  // ---- out = O / l
  {
    const int r0 = lane >> 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = r0 + 8 * half;
      if (row_pos[row] < 0) continue;
      const int tl = row / hpc, h = hb * 16 + row % hpc;
      const float inv = 1.0f / row_l[row];
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(a.out) + (start + tl0 + tl) * a.o_tok + h * a.o_head;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int c = col0 + i * 8 + (lane & 3) * 2;
        orow[c] = __float2bfloat16_rn(acc[i][2 * half] * inv);
        orow[c + 1] = __float2bfloat16_rn(acc[i][2 * half + 1] * inv);
      }
    }
  }
}

template <int NW, int NT>
static cudaError_t launch_latent_mma(const LatentAttnArgs& a, const LatentMmaSmem& sm, dim3 grid, cudaStream_t st) {
  auto kern = latent_attn_mma_kernel<NW, NT>;
  if (sm.total > 48 * 1024) {
    static bool raised = false;                  // one attribute per kernel instance: raise it to the card's limit once
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return e;
      raised = true;
    }
  }
  kern<<<grid, NW * 32, sm.total, st>>>(a, sm);
  return cudaSuccess;
}

// Sizes the tensor-core kernel takes: r a multiple of 32 (four or eight warps own whole 8-column tiles of O, at most
// eight each), dr a multiple of 8, everything addressable by 16-byte copies, one tile pair within shared memory.
static bool latent_mma_fits(const LatentAttnArgs& a, int* nw, int* nt) {
  if (a.r % 8 || a.dr % 8) return false;
  const int tiles = a.r / 8;
  if (tiles % 8 == 0 && tiles / 8 <= 8) { *nw = 8; *nt = tiles / 8; }
  else if (tiles % 4 == 0 && tiles / 4 <= 8) { *nw = 4; *nt = tiles / 4; }
  else return false;
  if (latent_mma_smem(a.r, a.dr).total > 220 * 1024) return false;
  if (reinterpret_cast<uintptr_t>(a.cache) % 16) return false;
  if (a.rot_dims % 2 || (a.dr % 2)) return false;
  return true;
}

static cudaError_t run_latent_mma(const LatentAttnArgs& a, int nw, int nt, cudaStream_t st) {
  const LatentMmaSmem sm = latent_mma_smem(a.r, a.dr);
  const int hpc = a.H < 16 ? a.H : 16, hblocks = (a.H + 15) / 16, G = 16 / hpc;
  const dim3 grid(static_cast<unsigned>((a.max_new + G - 1) / G) * hblocks, a.n_seqs);
#define LM_GO(NW, NT) return launch_latent_mma<NW, NT>(a, sm, grid, st)
#define LM_NT(NW) switch (nt) { case 1: LM_GO(NW, 1); case 2: LM_GO(NW, 2); case 3: LM_GO(NW, 3); case 4: LM_GO(NW, 4); \
                                case 5: LM_GO(NW, 5); case 6: LM_GO(NW, 6); case 7: LM_GO(NW, 7); case 8: LM_GO(NW, 8); }
  if (nw == 8) { LM_NT(8) } else { LM_NT(4) }
#undef LM_NT
#undef LM_GO
  return cudaErrorInvalidValue;
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
  int nw = 0, nt = 0;
  const bool fits = dtype == B2TTS_DTYPE_BF16 && latent_mma_fits(a, &nw, &nt);
  B2_REQUIRE(path != 2 || fits, B2TTS_EUNSUPPORTED, "latent_attn: the tensor-core kernel does not take kv_rank %d, rot_dim %d", kv_rank, rot_dim);
  if (fits && path != 1) {
    cudaError_t e = run_latent_mma(a, nw, nt, st);
    if (e != cudaSuccess) return cuda_fail(e, "latent_attn (tensor)");
    B2_CHECK_LAUNCH("latent_attn (tensor)");
    return B2TTS_OK;
  }
  const size_t smem = static_cast<size_t>(LA_WARPS) * (kv_rank + rot_dim) * sizeof(float);
  B2_REQUIRE(smem <= 48 * 1024, B2TTS_EUNSUPPORTED, "latent_attn: key size %d too large", kv_rank + rot_dim);
  const dim3 grid((static_cast<unsigned>(max_new) * heads + LA_WARPS - 1) / LA_WARPS, n_seqs);
  if (dtype == B2TTS_DTYPE_BF16) latent_attn_kernel<__nv_bfloat16><<<grid, LA_WARPS * 32, smem, st>>>(a);
  else latent_attn_kernel<float><<<grid, LA_WARPS * 32, smem, st>>>(a);
  B2_CHECK_LAUNCH("latent_attn");
  return B2TTS_OK;
}
