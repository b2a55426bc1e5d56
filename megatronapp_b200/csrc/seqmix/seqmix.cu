// Sequence-mixing kernels over a packed token batch (sm_100a): fp32-residual RMS norms, short causal convolution with a
// carried window, gated delta-rule and mLSTM matrix-memory scans, latent attention over a paged cache, group-limited router.
//
// Conventions: activations are `T` (float or __nv_bfloat16); statistics, gates, decays, scores and every recurrent state are
// fp32.  `cu[R + 1]` holds the sequence boundaries of the packed batch, `rows[R]` the state row of every sequence.
// The scans keep one column of the d x dv memory per thread in registers (columns never interact), stage q / k / gates of a
// chunk of tokens in shared memory, and therefore synchronise a few times per chunk instead of per token.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "seqmix_api.h"

namespace b200seq {

namespace {

template <typename T> __device__ __forceinline__ float ld(const T* p);
template <> __device__ __forceinline__ float ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st(T* p, float v);
template <> __device__ __forceinline__ void st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------------------------------------------
// x (fp32, in place) += delta ; y = x * rsqrt(mean(x^2) + eps) * w
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) add_rms_norm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                           const T* __restrict__ w, T* __restrict__ y, int cols, float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = x[base + c];
    if (delta != nullptr) {
      v += ld(delta + base + c);
      x[base + c] = v;
    }
    row[c] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  const float r = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) st(y + base + c, row[c] * r * ld(w + c));
}

// one warp per (token, head): o / rms(o) * w * sigmoid(gate)
template <typename T>
__global__ void gated_head_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ w, const T* __restrict__ gate,
                                           T* __restrict__ y, int n_rows, int H, int dv, int w_per_head, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31, h = row % H;
  const float* src = o + static_cast<int64_t>(row) * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
  for (int c = lane; c < dv; c += 32) {
    float v = src[c] * r * ld(w + (w_per_head ? h * dv : 0) + c);
    if (gate != nullptr) v *= sigmoidf_(ld(gate + static_cast<int64_t>(row) * dv + c));
    st(y + static_cast<int64_t>(row) * dv + c, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// depth-wise causal convolution + SiLU; the window holds the taps - 1 inputs that preceded the step
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w, const int* __restrict__ cu,
                                        const int* __restrict__ rows, const int* __restrict__ tok_seq, const T* __restrict__ window,
                                        T* __restrict__ y, int n_tok, int C, int taps) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(n_tok) * C) return;
  const int t = static_cast<int>(idx / C), c = static_cast<int>(idx % C);
  const int r = tok_seq[t], a = cu[r];
  const T* win = window + static_cast<int64_t>(rows[r]) * (taps - 1) * C;
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = t - (taps - 1 - j);
    const float in = src >= a ? ld(x + src * ldx + c) : ld(win + static_cast<int64_t>(taps - 1 + (src - a)) * C + c);
    acc += ld(w + static_cast<int64_t>(c) * taps + j) * in;
  }
  st(y + static_cast<int64_t>(t) * C + c, acc * sigmoidf_(acc));
}

template <typename T>
__global__ void conv_window_update_kernel(const T* __restrict__ x, int64_t ldx, const int* __restrict__ cu,
                                          const int* __restrict__ rows, T* __restrict__ window, int R, int C, int taps) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(R) * C) return;
  const int r = static_cast<int>(idx / C), c = static_cast<int>(idx % C);
  const int a = cu[r], b = cu[r + 1], n = b - a, keep = taps - 1;
  T* win = window + static_cast<int64_t>(rows[r]) * keep * C;
  for (int i = 0; i < keep; ++i) {                  // ascending: entry i + n is read before it can be overwritten
    const int src = b - keep + i;
    win[static_cast<int64_t>(i) * C + c] = src >= a ? x[src * ldx + c] : win[static_cast<int64_t>(i + n) * C + c];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// gated delta rule.  grid (column blocks, heads, sequences); thread j owns column j of S.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kChunk = 16;     // tokens staged per shared-memory round
constexpr int kCols = 64;      // columns (threads) per CTA

template <typename T, int D>
__global__ void __launch_bounds__(kCols) delta_rule_scan_kernel(DeltaArgs p) {
  __shared__ float sq[kChunk][D], sk[kChunk][D], sg[kChunk][D];
  __shared__ float sbeta[kChunk];
  const int h = blockIdx.y, r = blockIdx.z, kh = h / (p.H / p.KH);
  const int col = blockIdx.x * kCols + threadIdx.x;
  const bool live = col < p.dv;
  const int a = p.cu[r], b = p.cu[r + 1];
  if (a >= b) return;
  float* state = p.state + (static_cast<int64_t>(p.rows[r]) * p.H + h) * p.d * p.dv;
  float S[D];
#pragma unroll
  for (int i = 0; i < D; ++i) S[i] = (live && i < p.d) ? state[static_cast<int64_t>(i) * p.dv + col] : 0.f;
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kCols >> 5;
  for (int t0 = a; t0 < b; t0 += kChunk) {
    const int nt = min(kChunk, b - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * D; e += kCols) {
      const int tt = e / D, i = e % D, t = t0 + tt;
      const bool in = i < p.d;
      sq[tt][i] = in ? ld(q + t * p.ldq + kh * p.d + i) : 0.f;
      sk[tt][i] = in ? ld(k + t * p.ldk + kh * p.d + i) : 0.f;
      sg[tt][i] = in ? expf(p.log_decay[(static_cast<int64_t>(t) * p.H + h) * p.d + i]) : 1.f;
    }
    if (threadIdx.x < nt) sbeta[threadIdx.x] = p.beta[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {     // unit length (and the query's scale)
      float qq = 0.f, kk = 0.f;
      for (int i = lane; i < D; i += 32) { qq += sq[tt][i] * sq[tt][i]; kk += sk[tt][i] * sk[tt][i]; }
      qq = warp_sum(qq); kk = warp_sum(kk);
      const float rq = (p.unit_eps >= 0.f ? 1.0f / sqrtf(qq + p.unit_eps) : 1.0f) * p.q_scale;
      const float rk = p.unit_eps >= 0.f ? 1.0f / sqrtf(kk + p.unit_eps) : 1.0f;
      for (int i = lane; i < D; i += 32) { sq[tt][i] *= rq; sk[tt][i] *= rk; }
    }
    __syncthreads();
    if (live) {
#pragma unroll 1
      for (int tt = 0; tt < nt; ++tt) {
        const int t = t0 + tt;
        const float vv = ld(v + t * p.ldv + h * p.dv + col);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) { S[i] *= sg[tt][i]; acc = fmaf(S[i], sk[tt][i], acc); }
        const float u = sbeta[tt] * (vv - acc);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) { S[i] = fmaf(sk[tt][i], u, S[i]); o = fmaf(S[i], sq[tt][i], o); }
        p.out[(static_cast<int64_t>(t) * p.H + h) * p.dv + col] = o;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i < p.d) state[static_cast<int64_t>(i) * p.dv + col] = S[i];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// mLSTM.  Same layout; the normaliser n (a d-vector) and the running maximum m are advanced by every column block of a
// head (they do not depend on the columns) and written back by the first one.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kCols) mlstm_scan_kernel(MlstmArgs p) {
  __shared__ float sq[kChunk][D], sk[kChunk][D], sp[kChunk][D];
  __shared__ float skeep[kChunk], sput[kChunk], sfloor[kChunk], sden[kChunk];
  constexpr int NPT = (D + kCols - 1) / kCols;     // normaliser entries per thread
  const int h = blockIdx.y, r = blockIdx.z;
  const int col = blockIdx.x * kCols + threadIdx.x;
  const bool live = col < p.dv;
  const int a = p.cu[r], b = p.cu[r + 1];
  if (a >= b) return;
  const int64_t row = p.rows[r];
  float* state = p.state + (row * p.H + h) * p.d * p.dv;
  float* nstate = p.norm_state + (row * p.H + h) * p.d;
  float S[D], nvec[NPT];
#pragma unroll
  for (int i = 0; i < D; ++i) S[i] = (live && i < p.d) ? state[static_cast<int64_t>(i) * p.dv + col] : 0.f;
#pragma unroll
  for (int e = 0; e < NPT; ++e) {
    const int i = threadIdx.x + e * kCols;
    nvec[e] = (i < p.d) ? nstate[i] : 0.f;
  }
  float m = p.max_state[row * p.H + h];
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kCols >> 5;
  for (int t0 = a; t0 < b; t0 += kChunk) {
    const int nt = min(kChunk, b - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * D; e += kCols) {
      const int tt = e / D, i = e % D, t = t0 + tt;
      const bool in = i < p.d;
      sq[tt][i] = in ? ld(q + t * p.ldq + h * p.d + i) * p.q_scale : 0.f;
      sk[tt][i] = in ? ld(k + t * p.ldk + h * p.d + i) : 0.f;
    }
    if (threadIdx.x == 0) {                          // the gate recurrence is scalar: one thread walks the chunk
      float mm = m;
      for (int tt = 0; tt < nt; ++tt) {
        const float li = p.log_i[static_cast<int64_t>(t0 + tt) * p.H + h], lf = p.log_f[static_cast<int64_t>(t0 + tt) * p.H + h];
        const float m_new = fmaxf(lf + mm, li);
        skeep[tt] = expf(lf + mm - m_new);
        sput[tt] = expf(li - m_new);
        sfloor[tt] = expf(-m_new);
        mm = m_new;
      }
      sden[0] = mm;
    }
    __syncthreads();
    m = sden[0];
    // normaliser: n <- keep n + put k, and the products n_i q_i of every token of the chunk
    for (int tt = 0; tt < nt; ++tt) {
#pragma unroll
      for (int e = 0; e < NPT; ++e) {
        const int i = threadIdx.x + e * kCols;
        if (i < D) {
          nvec[e] = skeep[tt] * nvec[e] + sput[tt] * sk[tt][i];
          sp[tt][i] = nvec[e] * sq[tt][i];
        }
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {
      float s = 0.f;
      for (int i = lane; i < D; i += 32) s += sp[tt][i];
      s = warp_sum(s);
      if (lane == 0) sden[tt] = fmaxf(fabsf(s), sfloor[tt]) + p.denom_eps;
    }
    __syncthreads();
    if (live) {
#pragma unroll 1
      for (int tt = 0; tt < nt; ++tt) {
        const int t = t0 + tt;
        const float pv = sput[tt] * ld(v + t * p.ldv + h * p.dv + col), keep = skeep[tt];
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) { S[i] = fmaf(keep, S[i], sk[tt][i] * pv); o = fmaf(S[i], sq[tt][i], o); }
        p.out[(static_cast<int64_t>(t) * p.H + h) * p.dv + col] = o / sden[tt];
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i < p.d) state[static_cast<int64_t>(i) * p.dv + col] = S[i];
  }
  if (blockIdx.x == 0) {
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
      const int i = threadIdx.x + e * kCols;
      if (i < p.d) nstate[i] = nvec[e];
    }
    if (threadIdx.x == 0) p.max_state[row * p.H + h] = m;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// latent attention over paged latents.  grid (tokens, head groups); each warp walks a strided subset of the visible keys
// with an online softmax per head, the warps' partial results are merged through shared memory.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kAttnWarps = 4;

template <typename T, int RPL, int HG>
__global__ void __launch_bounds__(kAttnWarps * 32) latent_attention_kernel(LatentAttnArgs p) {
  extern __shared__ float smem[];                   // q [HG][r] | per warp: m [HG], l [HG], acc [HG][r]
  const int t = blockIdx.x, h0 = blockIdx.y * HG, nh = min(HG, p.H - h0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = p.r, len = p.tok_len[t];
  const int* table = p.block_table + static_cast<int64_t>(p.tok_req[t]) * p.max_blocks;
  float* sq = smem;
  float* part = smem + HG * r;
  const T* q = static_cast<const T*>(p.q) + (static_cast<int64_t>(t) * p.H + h0) * r;
  for (int e = threadIdx.x; e < HG * r; e += blockDim.x) sq[e] = (e / r) < nh ? ld(q + e) * p.scale : 0.f;
  __syncthreads();
  float mx[HG], l[HG], acc[HG][RPL];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    mx[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < RPL; ++e) acc[g][e] = 0.f;
  }
  const T* cache = static_cast<const T*>(p.cache);
  for (int j = warp; j < len; j += kAttnWarps) {
    const int64_t slot = static_cast<int64_t>(table[j / p.block_size]) * p.block_size + j % p.block_size;
    float c[RPL];
#pragma unroll
    for (int e = 0; e < RPL; ++e) {
      const int i = lane + 32 * e;
      c[e] = i < r ? ld(cache + slot * r + i) : 0.f;
    }
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < RPL; ++e) {
        const int i = lane + 32 * e;
        if (i < r) s = fmaf(sq[g * r + i], c[e], s);
      }
      s = warp_sum(s);
      const float m_new = fmaxf(mx[g], s);
      const float corr = expf(mx[g] - m_new), w = expf(s - m_new);
      l[g] = l[g] * corr + w;
#pragma unroll
      for (int e = 0; e < RPL; ++e) acc[g][e] = acc[g][e] * corr + w * c[e];
      mx[g] = m_new;
    }
  }
  float* mine = part + static_cast<int64_t>(warp) * HG * (r + 2);
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) { mine[g * (r + 2)] = mx[g]; mine[g * (r + 2) + 1] = l[g]; }
#pragma unroll
    for (int e = 0; e < RPL; ++e) {
      const int i = lane + 32 * e;
      if (i < r) mine[g * (r + 2) + 2 + i] = acc[g][e];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < nh * r; e += blockDim.x) {
    const int g = e / r, i = e % r;
    float m_all = -INFINITY;
    for (int w = 0; w < kAttnWarps; ++w) m_all = fmaxf(m_all, part[(w * HG + g) * (r + 2)]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* pw = part + (w * HG + g) * (r + 2);
      const float f = pw[0] == -INFINITY ? 0.f : expf(pw[0] - m_all);
      num += f * pw[2 + i];
      den += f * pw[1];
    }
    p.out[(static_cast<int64_t>(t) * p.H + h0 + g) * r + i] = num / den;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// router: one warp per token
// ---------------------------------------------------------------------------------------------------------------------
__global__ void group_limited_router_kernel(const float* __restrict__ logits, float* __restrict__ probs, bool* __restrict__ rmap,
                                            int n_tok, int E, int topk, int G, int keep, int renorm) {
  extern __shared__ float smem[];                   // per warp: scores [E], group best [G]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tok) return;
  float* s = smem + static_cast<int64_t>(warp) * (E + G);
  float* gbest = s + E;
  const float* z = logits + static_cast<int64_t>(t) * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - mx); s[e] = v; sum += v; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  __syncwarp();
  const int per = E / G;
  for (int g = lane; g < G; g += 32) {
    float b = -1.f;
    for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, s[e]);
    gbest[g] = b;
  }
  __syncwarp();
  // drop all but the `keep` best groups: repeatedly take the best remaining group and mark it (score + 2 > 1)
  for (int it = 0; it < keep; ++it) {
    float bv = -1.f; int bi = 0x7fffffff;
    for (int g = lane; g < G; g += 32) {
      const float v = gbest[g];
      if (v <= 1.5f && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0 && bi < G) gbest[bi] += 2.f;
    __syncwarp();
  }
  float wsum = 0.f;
  int chosen[32];                                   // topk <= 32 (checked on the host)
  for (int it = 0; it < topk; ++it) {
    float bv = -1.f; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s[e];
      if (v >= 0.f && gbest[e / per] > 1.5f && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    chosen[it] = bi;
    if (bi < E) {
      wsum += bv;
      if (lane == 0) { probs[static_cast<int64_t>(t) * E + bi] = bv; s[bi] = -1.f; }
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = renorm ? 1.0f / (wsum + 1e-20f) : 1.0f;
    for (int it = 0; it < topk; ++it)
      if (chosen[it] < E) {
        probs[static_cast<int64_t>(t) * E + chosen[it]] *= inv;
        rmap[static_cast<int64_t>(t) * E + chosen[it]] = true;
      }
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
#define SEQ_DISPATCH_T(is_bf16, ...)                      \
  if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else { using T = float; __VA_ARGS__; }

void add_rms_norm(float* x, const void* delta, const void* w, void* y, int rows, int cols, float eps, bool bf16, cudaStream_t s) {
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, add_rms_norm_kernel<T><<<rows, 256, cols * sizeof(float), s>>>(
                           x, static_cast<const T*>(delta), static_cast<const T*>(w), static_cast<T*>(y), cols, eps));
}

void gated_head_rms_norm(const float* o, const void* w, const void* gate, void* y, int n_tok, int H, int dv, bool w_per_head,
                         float eps, bool bf16, cudaStream_t s) {
  const int rows = n_tok * H;
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, gated_head_rms_norm_kernel<T><<<(rows + 3) / 4, 128, 0, s>>>(
                           o, static_cast<const T*>(w), static_cast<const T*>(gate), static_cast<T*>(y), rows, H, dv,
                           w_per_head ? 1 : 0, eps));
}

void causal_conv_silu(const void* x, int64_t ldx, const void* w, const int* cu, const int* rows, const int* tok_seq, void* window,
                      void* y, int n_tok, int R, int C, int taps, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return;
  const int64_t n = static_cast<int64_t>(n_tok) * C;
  SEQ_DISPATCH_T(bf16, {
    causal_conv_silu_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
        static_cast<const T*>(x), ldx, static_cast<const T*>(w), cu, rows, tok_seq, static_cast<const T*>(window),
        static_cast<T*>(y), n_tok, C, taps);
    if (taps > 1)
      conv_window_update_kernel<T><<<(R * C + 255) / 256, 256, 0, s>>>(static_cast<const T*>(x), ldx, cu, rows,
                                                                        static_cast<T*>(window), R, C, taps);
  });
}

template <typename T>
static bool launch_delta(const DeltaArgs& p, dim3 grid, cudaStream_t s) {
  if (p.d <= 32) delta_rule_scan_kernel<T, 32><<<grid, kCols, 0, s>>>(p);
  else if (p.d <= 64) delta_rule_scan_kernel<T, 64><<<grid, kCols, 0, s>>>(p);
  else if (p.d <= 128) delta_rule_scan_kernel<T, 128><<<grid, kCols, 0, s>>>(p);
  else return false;
  return true;
}

bool delta_rule_scan(const DeltaArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  dim3 grid((p.dv + kCols - 1) / kCols, p.H, R);
  return bf16 ? launch_delta<__nv_bfloat16>(p, grid, s) : launch_delta<float>(p, grid, s);
}

template <typename T>
static bool launch_mlstm(const MlstmArgs& p, dim3 grid, cudaStream_t s) {
  if (p.d <= 32) mlstm_scan_kernel<T, 32><<<grid, kCols, 0, s>>>(p);
  else if (p.d <= 64) mlstm_scan_kernel<T, 64><<<grid, kCols, 0, s>>>(p);
  else if (p.d <= 128) mlstm_scan_kernel<T, 128><<<grid, kCols, 0, s>>>(p);
  else return false;
  return true;
}

bool mlstm_scan(const MlstmArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  dim3 grid((p.dv + kCols - 1) / kCols, p.H, R);
  return bf16 ? launch_mlstm<__nv_bfloat16>(p, grid, s) : launch_mlstm<float>(p, grid, s);
}

template <typename T, int RPL, int HG>
static bool launch_attn(const LatentAttnArgs& p, int n_tok, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(HG) * p.r + static_cast<size_t>(kAttnWarps) * HG * (p.r + 2)) * sizeof(float);
  auto kern = latent_attention_kernel<T, RPL, HG>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return false;
  dim3 grid(n_tok, (p.H + HG - 1) / HG);
  kern<<<grid, kAttnWarps * 32, smem, s>>>(p);
  return true;
}

template <typename T>
static bool dispatch_attn(const LatentAttnArgs& p, int n_tok, cudaStream_t s) {
  const int rpl = (p.r + 31) / 32;                  // latent entries per lane; heads per CTA shrink as it grows
  if (rpl <= 2) return p.H >= 8 ? launch_attn<T, 2, 8>(p, n_tok, s) : launch_attn<T, 2, 4>(p, n_tok, s);
  if (rpl <= 4) return p.H >= 8 ? launch_attn<T, 4, 8>(p, n_tok, s) : launch_attn<T, 4, 4>(p, n_tok, s);
  if (rpl <= 8) return launch_attn<T, 8, 4>(p, n_tok, s);
  if (rpl <= 16) return launch_attn<T, 16, 2>(p, n_tok, s);
  if (rpl <= 32) return launch_attn<T, 32, 1>(p, n_tok, s);
  return false;
}

bool latent_attention_paged(const LatentAttnArgs& p, int n_tok, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return true;
  return bf16 ? dispatch_attn<__nv_bfloat16>(p, n_tok, s) : dispatch_attn<float>(p, n_tok, s);
}

bool group_limited_router(const float* logits, float* probs, bool* rmap, int n_tok, int E, int topk, int G, int keep, bool renorm,
                          cudaStream_t s) {
  if (n_tok == 0) return true;
  if (topk > 32 || G <= 0 || E % G != 0) return false;
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * (E + G) * sizeof(float);
  if (smem > 48 * 1024) return false;
  group_limited_router_kernel<<<(n_tok + warps - 1) / warps, warps * 32, smem, s>>>(logits, probs, rmap, n_tok, E, topk, G, keep,
                                                                                   renorm ? 1 : 0);
  return true;
}

}  // namespace b200seq
