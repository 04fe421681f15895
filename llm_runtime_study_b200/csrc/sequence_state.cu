// Mixers that carry a state of fixed size per request instead of a growing cache:
//
//   linear scan     S_t = D_t S_(t-1) + k_t u_t^T,  o_t = S_t^T q_t        per head, S is [d, dv]
//                   (the delta rule's read-out is formed as (D_t S_(t-1))^T q_t + u_t (k_t . q_t), the same sum)
//                   D_t = one decay per head (a constant), or a diagonal of per-row factors g_t (gated)
//                   u_t = v_t (plain), or beta_t (v_t - (D_t S_(t-1))^T k_t) (delta rule)
//   short convolution over time per channel, with the last taps-1 inputs kept per request
//   per-group RMS norm of the read-out times a sigmoid gate
//
// The state, the decays, the gates of the recurrence and the unit norms are float32 whatever the
// storage type of the projections.  Tokens of one request are processed in order, one after the
// other, from the state the request's slot holds, so a token's result does not depend on how the
// sequence was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// SiLU of a value that was stored in 16 bits: the hardware's exponential and reciprocal are exact far beyond the
// 8 bits of such a value; 32-bit inputs take the full-precision functions.
template <typename T> __device__ __forceinline__ float silu_of(float x) {
  if constexpr (sizeof(T) == 2) return __fdividef(x, 1.f + __expf(-x));
  else return silu_f(x);
}

// ---------------------------------------------------------------------------- linear scan
struct ScanParams {
  const void* q; const void* k; const void* v;   // rows of the storage type; heads side by side
  int ldq, ldk, ldv;                              // row strides in elements
  const float* gate; int ldg;                     // [n, H * d] per-row factors (gated) or null
  const float* decay;                             // [H] constant factors (not gated)
  const float* beta; int ldb;                     // [n, H] (delta rule) or null
  float* state;                                   // [slots, H, d, dv]
  float* out; int ldo;                            // [n, H * dv]
  const int* q_start; const int* slots;           // per entry: first token, request slot
  int H, Hqk, d, dv, act, rl;                     // act 1: silu on q, k, v as they are read; rl: lanes that share a column
};

constexpr int kScanThreads = 128;
// tokens staged in shared memory at a time: 16, or 8 where a token's rows are more than 128 wide
constexpr int scan_chunk(int dpt, int rl) { return dpt * rl <= 128 ? 16 : 8; }

// One CTA owns some columns of one head's state for one request.  A column is independent of the
// others: S[:, c] <- D S[:, c] + k u_c.  Its d rows are spread over RL lanes of one warp (lane r
// owns rows r * DPT .. r * DPT + DPT - 1, so that it reads its part of k, q and g from shared memory
// 16 bytes at a time), DPT rows per lane in registers; the two dot products over rows are finished
// by shuffles.  RL = 4 keeps 8 neighbouring columns (one 32-byte sector of a state row) in
// a warp, which is what a launch that mostly moves states wants (many requests, one token each);
// RL = 16 spreads a column over more lanes and a head over sixteen times as many CTAs, which is
// what a launch with few requests and long portions wants: its time is a chain of dependent steps,
// and the chain per token is a quarter as long.
template <typename T, int DPT, int RL, bool DELTA, bool GATED>
__global__ void __launch_bounds__(kScanThreads) linear_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  constexpr int rl = RL, cols_per_warp = 32 / rl, cols = (kScanThreads / 32) * cols_per_warp;
  constexpr int dp = DPT * rl;                          // rows padded to dp >= d; the padding holds zeros
  constexpr int CHUNK = scan_chunk(DPT, RL);            // tokens staged in shared memory at a time
  constexpr int EPT = CHUNK * dp / kScanThreads;        // staged elements of k (q, g) per thread
  constexpr int VPT = (CHUNK * cols + kScanThreads - 1) / kScanThreads;
  const int col_blocks = (p.dv + cols - 1) / cols;
  const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks;
  const int entry = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane / cols_per_warp;
  const int col_local = warp * cols_per_warp + lane % cols_per_warp;
  const int col = cb * cols + col_local;
  const bool live = col < p.dv;
  const int d = p.d, dv = p.dv;
  const int hqk = h / (p.H / p.Hqk);
  const int t_begin = p.q_start[entry], t_end = p.q_start[entry + 1];
  const int slot = p.slots[entry];
  float* sbase = p.state + (static_cast<size_t>(slot) * p.H + h) * d * dv;

  float* ks = smem;                              // [chunk][dp]
  float* qs = ks + CHUNK * dp;                   // [chunk][dp]
  float* gs = qs + CHUNK * dp;                   // [chunk][dp] (gated only)
  float* vs = gs + (GATED ? CHUNK * dp : 0);     // [chunk][cols]
  float* bs = vs + CHUNK * cols;                 // [chunk]
  const float dec = GATED ? 1.f : p.decay[h];
  const T* qg = static_cast<const T*>(p.q);
  const T* kg = static_cast<const T*>(p.k);
  const T* vg = static_cast<const T*>(p.v);

  // The rows of the next chunk are asked for before the tokens of this one are worked through, and land in
  // registers; they go to shared memory (SiLU applied once per element) when this chunk is done.
  // (kept in the storage type: a conversion right behind the load would wait for it)
  T rk[EPT], rq[EPT], rv[VPT];
  float rg[EPT], rb = 0.f;
  auto fetch = [&](int t0, int count) {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      if (e * kScanThreads >= count * dp) break;       // a single decoded token fills one round, not sixteen
      const int idx = threadIdx.x + e * kScanThreads;
      const int tt = idx / dp, i = idx % dp;
      rk[e] = rq[e] = from_float<T>(0.f);
      rg[e] = 0.f;
      if (tt < count && i < d) {
        const size_t row = static_cast<size_t>(t0 + tt);
        rk[e] = kg[row * p.ldk + hqk * d + i];
        rq[e] = qg[row * p.ldq + hqk * d + i];
        if (GATED) rg[e] = p.gate[row * p.ldg + h * d + i];
      }
    }
#pragma unroll
    for (int e = 0; e < VPT; ++e) {
      if (e * kScanThreads >= count * cols) break;
      const int idx = threadIdx.x + e * kScanThreads;
      const int tt = idx / cols, c = cb * cols + idx % cols;
      rv[e] = (tt < count && c < dv) ? vg[static_cast<size_t>(t0 + tt) * p.ldv + h * dv + c] : from_float<T>(0.f);
    }
    if (DELTA && threadIdx.x < count) rb = p.beta[static_cast<size_t>(t0 + threadIdx.x) * p.ldb + h];
  };
  auto stash = [&](int count) {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      if (e * kScanThreads >= count * dp) break;
      const int idx = threadIdx.x + e * kScanThreads;
      ks[idx] = p.act ? silu_of<T>(to_float(rk[e])) : to_float(rk[e]);
      qs[idx] = p.act ? silu_of<T>(to_float(rq[e])) : to_float(rq[e]);
      if (GATED) gs[idx] = rg[e];
    }
#pragma unroll
    for (int e = 0; e < VPT; ++e) {
      if (e * kScanThreads >= count * cols) break;
      const int idx = threadIdx.x + e * kScanThreads;
      if (idx < CHUNK * cols) vs[idx] = p.act ? silu_of<T>(to_float(rv[e])) : to_float(rv[e]);
    }
    if (DELTA && threadIdx.x < CHUNK) bs[threadIdx.x] = rb;
  };

  fetch(t_begin, min(CHUNK, t_end - t_begin));
  float S[DPT];
#pragma unroll
  for (int ii = 0; ii < DPT; ++ii) {
    const int i = r * DPT + ii;
    S[ii] = (live && i < d) ? sbase[static_cast<size_t>(i) * dv + col] : 0.f;
  }

  for (int t0 = t_begin; t0 < t_end; t0 += CHUNK) {
    const int count = min(CHUNK, t_end - t0);
    __syncthreads();            // every warp is through the chunk before
    stash(count);
    __syncthreads();
    if (t0 + CHUNK < t_end) fetch(t0 + CHUNK, min(CHUNK, t_end - t0 - CHUNK));
    for (int tt = 0; tt < count; ++tt) {
      const float4* kt = reinterpret_cast<const float4*>(ks + tt * dp + r * DPT);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * dp + r * DPT);
      const float4* gt = reinterpret_cast<const float4*>(gs + tt * dp + r * DPT);
      float4 kk[DPT / 4];
      float o_sum;
      if constexpr (DELTA) {
        // o = (D S)^T q + u (k . q): the three sums over rows (against k, against q, and k . q) are formed in one
        // pass and reduced over the lanes together, so a token costs one shuffle tree, not two in a row
        float dot[2] = {0.f, 0.f}, oq[2] = {0.f, 0.f}, kq[2] = {0.f, 0.f};
#pragma unroll
        for (int v = 0; v < DPT / 4; ++v) {
          kk[v] = kt[v];
          const float4 qq = qt[v];
          if (GATED) {
            const float4 g = gt[v];
            S[4 * v] *= g.x; S[4 * v + 1] *= g.y; S[4 * v + 2] *= g.z; S[4 * v + 3] *= g.w;
          } else {
            S[4 * v] *= dec; S[4 * v + 1] *= dec; S[4 * v + 2] *= dec; S[4 * v + 3] *= dec;
          }
          dot[0] = fmaf(S[4 * v], kk[v].x, dot[0]);
          dot[1] = fmaf(S[4 * v + 1], kk[v].y, dot[1]);
          dot[0] = fmaf(S[4 * v + 2], kk[v].z, dot[0]);
          dot[1] = fmaf(S[4 * v + 3], kk[v].w, dot[1]);
          oq[0] = fmaf(S[4 * v], qq.x, oq[0]);
          oq[1] = fmaf(S[4 * v + 1], qq.y, oq[1]);
          oq[0] = fmaf(S[4 * v + 2], qq.z, oq[0]);
          oq[1] = fmaf(S[4 * v + 3], qq.w, oq[1]);
          kq[0] = fmaf(kk[v].x, qq.x, kq[0]);
          kq[1] = fmaf(kk[v].y, qq.y, kq[1]);
          kq[0] = fmaf(kk[v].z, qq.z, kq[0]);
          kq[1] = fmaf(kk[v].w, qq.w, kq[1]);
        }
        float sum = dot[0] + dot[1], sq_ = oq[0] + oq[1], skq = kq[0] + kq[1];
#pragma unroll
        for (int o = cols_per_warp; o < 32; o <<= 1) {
          sum += __shfl_xor_sync(0xffffffffu, sum, o);
          sq_ += __shfl_xor_sync(0xffffffffu, sq_, o);
          skq += __shfl_xor_sync(0xffffffffu, skq, o);
        }
        const float u = bs[tt] * (vs[tt * cols + col_local] - sum);
        o_sum = fmaf(u, skq, sq_);
#pragma unroll
        for (int v = 0; v < DPT / 4; ++v) {
          S[4 * v] = fmaf(kk[v].x, u, S[4 * v]);
          S[4 * v + 1] = fmaf(kk[v].y, u, S[4 * v + 1]);
          S[4 * v + 2] = fmaf(kk[v].z, u, S[4 * v + 2]);
          S[4 * v + 3] = fmaf(kk[v].w, u, S[4 * v + 3]);
        }
      } else {
        const float u = vs[tt * cols + col_local];
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int v = 0; v < DPT / 4; ++v) {
          kk[v] = kt[v];
          const float4 qq = qt[v];
          if (GATED) {
            const float4 g = gt[v];
            S[4 * v] *= g.x; S[4 * v + 1] *= g.y; S[4 * v + 2] *= g.z; S[4 * v + 3] *= g.w;
          } else {
            S[4 * v] *= dec; S[4 * v + 1] *= dec; S[4 * v + 2] *= dec; S[4 * v + 3] *= dec;
          }
          S[4 * v] = fmaf(kk[v].x, u, S[4 * v]);
          S[4 * v + 1] = fmaf(kk[v].y, u, S[4 * v + 1]);
          S[4 * v + 2] = fmaf(kk[v].z, u, S[4 * v + 2]);
          S[4 * v + 3] = fmaf(kk[v].w, u, S[4 * v + 3]);
          acc[0] = fmaf(S[4 * v], qq.x, acc[0]);
          acc[1] = fmaf(S[4 * v + 1], qq.y, acc[1]);
          acc[2] = fmaf(S[4 * v + 2], qq.z, acc[2]);
          acc[3] = fmaf(S[4 * v + 3], qq.w, acc[3]);
        }
        o_sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int o = cols_per_warp; o < 32; o <<= 1) o_sum += __shfl_xor_sync(0xffffffffu, o_sum, o);
      }
      if (live && r == 0) p.out[static_cast<size_t>(t0 + tt) * p.ldo + h * dv + col] = o_sum;
    }
  }
#pragma unroll
  for (int ii = 0; ii < DPT; ++ii) {
    const int i = r * DPT + ii;
    if (live && i < d) sbase[static_cast<size_t>(i) * dv + col] = S[ii];
  }
}

template <typename T, bool DELTA, bool GATED>
int launch_scan(ScanParams p, int entries, cudaStream_t stream) {
  const int dpt = (p.d + p.rl - 1) / p.rl;
  const int cols = (kScanThreads / 32) * (32 / p.rl);
  dim3 grid(p.H * ((p.dv + cols - 1) / cols), entries);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  const int dpt8 = (dpt + 7) / 8 * 8;
  const int chunk = scan_chunk(dpt8, p.rl);
  const size_t smem = sizeof(float) * (static_cast<size_t>(chunk) * dpt8 * p.rl * (GATED ? 3 : 2) + chunk * cols + chunk);
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
#define B200_SCAN_CASE(DPT_, RL_)                                                                                      \
  if (dpt8 == DPT_ && p.rl == RL_) {                                                                                   \
    launch(linear_scan_kernel<T, DPT_, RL_, DELTA, GATED>, grid, dim3(kScanThreads), smem, stream, p);                 \
    return launch_status();                                                                                            \
  }
  B200_SCAN_CASE(8, 4) B200_SCAN_CASE(16, 4) B200_SCAN_CASE(24, 4) B200_SCAN_CASE(32, 4)
  B200_SCAN_CASE(8, 8) B200_SCAN_CASE(16, 8) B200_SCAN_CASE(24, 8) B200_SCAN_CASE(32, 8)
  B200_SCAN_CASE(8, 16) B200_SCAN_CASE(16, 16)
#undef B200_SCAN_CASE
  return B200_ERR_TOO_LARGE;
}

// Lanes per column for a launch: 16 where the key size needs them (more than 128 rows) or where 4 would leave most
// of the GPU idle (fewer CTAs than two per SM); 4 otherwise.
static int scan_row_lanes(int entries, int H, int d, int dv, int tokens, int fixed_order) {
  if (d > 128) return 16;
  if (fixed_order) return 4;       // the order of a column's sums must not depend on the shape of the batch
  static int wide = -1;            // LLM_RUNTIME_STUDY_B200_SCAN_LANES: 8 or 16 lanes for launches with few long portions
  if (wide < 0) {
    const char* e = getenv("LLM_RUNTIME_STUDY_B200_SCAN_LANES");
    wide = (e && atoi(e) == 8) ? 8 : 16;
  }
  const int ctas4 = entries * H * ((dv + 31) / 32);
  return (ctas4 < 2 * 148 && tokens > entries) ? wide : 4;
}

// ---------------------------------------------- preparation of a gated delta rule's inputs
struct DeltaPrepareParams {
  const void* proj; int ld;        // [n, ld] stacked projection: q | k | v | beta | decay rank | ...
  int b_off, a_off, rank;          // columns of the beta logits and of the low-rank decay input
  const float* taps; int ntaps;    // [C, ntaps], C = 2 G d + H dv channels in the order q, k, v
  const float* conv_state;         // [slots, ntaps - 1, C]: inputs of the positions before this step, oldest first
  const float* a_log;              // [H]
  const float* dt_bias;            // [H d]
  const void* a_up;                // [rank, H d] storage type (the map's weight transposed: neighbouring threads read neighbouring outputs)
  float* q; float* k; float* v; float* g; float* beta;   // [n, G d], [n, G d], [n, H dv], [n, H d], [n, H]
  const int* q_start; const int* slots; const int* token_entry;
  int H, G, d, dv;
  float unit_eps, q_scale;
};

// One CTA per head and block of `tokens_per_cta` tokens (1 for small batches, so that a decode step spreads over
// heads x tokens CTAs; more for prompt portions, so that the head's taps and its slice of the low-rank map are
// fetched once per CTA into shared memory).  Per token: the convolution and SiLU of the head's value channels, of its
// q and k channels (the first head of a group of heads that share them does these), their unit norms, the head's
// decay factors g = exp(-exp(a_log) * softplus(low-rank(x) + dt_bias)), and beta = sigmoid(.).  Every sum has an
// order that depends on the sizes only.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const DeltaPrepareParams p, int n, int tokens_per_cta) {
  extern __shared__ float smem[];
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y;
  const int d = p.d, dv = p.dv, qk = p.G * d, C = 2 * qk + p.H * dv, K = p.ntaps;
  const int group = p.H / p.G, gq = h / group;
  const bool does_qk = h % group == 0;
  const T* proj = static_cast<const T*>(p.proj);
  const size_t hv = static_cast<size_t>(p.H) * dv, hd = static_cast<size_t>(p.H) * d;
  float* sq = smem;                    // [d]
  float* sk = sq + d;                  // [d]
  float* low = sk + d;                 // [rank]
  float* up_s = low + p.rank;          // [rank][d]: this head's slice of the low-rank map
  float* taps_s = up_s + p.rank * d;   // [(2 d + dv)][K]: taps of this head's q, k and v channels
  const T* up = static_cast<const T*>(p.a_up);
  for (int idx = threadIdx.x; idx < p.rank * d; idx += blockDim.x)
    up_s[idx] = to_float(up[static_cast<size_t>(idx / d) * hd + static_cast<size_t>(h) * d + idx % d]);
  for (int idx = threadIdx.x; idx < (2 * d + dv) * K; idx += blockDim.x) {
    const int lc = idx / K, j = idx % K;     // local channel: q [0, d), k [d, 2d), v [2d, 2d + dv)
    const int c = lc < d ? gq * d + lc : (lc < 2 * d ? qk + gq * d + (lc - d) : 2 * qk + h * dv + (lc - 2 * d));
    taps_s[idx] = p.taps[static_cast<size_t>(c) * K + j];
  }
  const float rate = expf(p.a_log[h]);
  const int t_end = min(n, (static_cast<int>(blockIdx.x) + 1) * tokens_per_cta);
  for (int t = blockIdx.x * tokens_per_cta; t < t_end; ++t) {
    const int entry = p.token_entry[t];
    const int first = p.q_start[entry];
    const int local = t - first;
    const int slot = p.slots[entry];
    auto conv = [&](int c, int lc) {
      float acc = 0.f;
      for (int j = 0; j < K; ++j) {
        const int at = local - (K - 1 - j);
        const float x = at >= 0 ? to_float(proj[static_cast<size_t>(first + at) * p.ld + c])
                                : p.conv_state[(static_cast<size_t>(slot) * (K - 1) + (K - 1 + at)) * C + c];
        acc = fmaf(taps_s[lc * K + j], x, acc);
      }
      return silu_of<T>(acc);
    };
    __syncthreads();             // the shared arrays are filled, and the token before is done with sq, sk and low
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x) low[i] = to_float(proj[static_cast<size_t>(t) * p.ld + p.a_off + i]);
    for (int i = threadIdx.x; i < dv; i += blockDim.x) p.v[t * hv + h * dv + i] = conv(2 * qk + h * dv + i, 2 * d + i);
    if (does_qk) {               // the same for every thread of the CTA
      float ssq = 0.f, ssk = 0.f;
      for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float a = conv(gq * d + i, i), b = conv(qk + gq * d + i, d + i);
        sq[i] = a;
        sk[i] = b;
        ssq = fmaf(a, a, ssq);
        ssk = fmaf(b, b, ssk);
      }
      const float fq = rsqrtf(block_sum(ssq, scratch) + p.unit_eps) * p.q_scale;
      const float fk = rsqrtf(block_sum(ssk, scratch) + p.unit_eps);
      for (int i = threadIdx.x; i < d; i += blockDim.x) {
        p.q[static_cast<size_t>(t) * qk + gq * d + i] = sq[i] * fq;
        p.k[static_cast<size_t>(t) * qk + gq * d + i] = sk[i] * fk;
      }
    }
    __syncthreads();             // low[] is complete
    if (threadIdx.x == 0) p.beta[static_cast<size_t>(t) * p.H + h] = sigmoid_f(to_float(proj[static_cast<size_t>(t) * p.ld + p.b_off + h]));
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const size_t col = static_cast<size_t>(h) * d + i;
      float a = 0.f;
      for (int j = 0; j < p.rank; ++j) a = fmaf(up_s[j * d + i], low[j], a);
      p.g[t * hd + col] = expf(-rate * softplus_f(a + p.dt_bias[col]));
    }
  }
}

// After a step: the last taps-1 inputs of each request, from the step's rows and, where the step
// was shorter than that, from what the state held.  One thread per channel walks the rows oldest
// first; row s is written after row len + s (> s) has been read, so nothing is read after it changed.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, float* __restrict__ conv_state, int C, int ntaps,
                                         const int* __restrict__ q_start, const int* __restrict__ slots) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int first = q_start[entry], len = q_start[entry + 1] - first;
  float* st = conv_state + static_cast<size_t>(slots[entry]) * (ntaps - 1) * C;
  for (int s = 0; s < ntaps - 1; ++s) {
    const int at = len - (ntaps - 1) + s;
    st[static_cast<size_t>(s) * C + c] = at >= 0 ? to_float(proj[static_cast<size_t>(first + at) * ld + c])
                                                 : st[static_cast<size_t>(len + s) * C + c];
  }
}

// ------------------------------------------------------------- group norm times sigmoid gate
// out[t, c] = x[t, c] * rsqrt(mean over c's group of x^2 + eps) * w[c % group] * sigmoid(gate[t, c]);
// the gate's logits are read from `gate_in` directly (rank 0) or formed as gate_up[:, c] . gate_in[t, :rank]
// (gate_up is [rank, width]: the map's weight transposed).
template <typename T>
__global__ void group_norm_gate_kernel(const float* __restrict__ x, int width, int group, const float* __restrict__ w, float eps,
                                       const T* __restrict__ gate_in, int gate_ld, int rank, const T* __restrict__ gate_up,
                                       T* __restrict__ out) {
  __shared__ float scratch[32];
  extern __shared__ float low[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, base = blockIdx.y * group;
  const float* row = x + static_cast<size_t>(t) * width + base;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) low[j] = to_float(gate_in[static_cast<size_t>(t) * gate_ld + j]);
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  const float f = rsqrtf(block_sum(ss, scratch) / static_cast<float>(group) + eps);
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const int c = base + i;
    float logit;
    if (rank == 0) {
      logit = to_float(gate_in[static_cast<size_t>(t) * gate_ld + c]);
    } else {
      logit = 0.f;
      for (int j = 0; j < rank; ++j) logit = fmaf(to_float(gate_up[static_cast<size_t>(j) * width + c]), low[j], logit);
    }
    out[static_cast<size_t>(t) * width + c] = from_float<T>(row[i] * f * w[i] * sigmoid_f(logit));
  }
}

}  // namespace b200

// `tokens`: rows in the batch (with `entries` it tells a batch of single tokens from one that holds portions).
// `fixed_order`: the same lanes per column whatever the batch looks like, so that a token's bits do not depend on the cut.
// q, k: [n, Hqk * d] rows (strides ldq, ldk), v: [n, H * dv]; element type by `dtype`.  gate (float32 [n, H * d]) selects
// per-row factors, else `decay` ([H]) is used; beta (float32 [n, H]) selects the delta rule.  state float32 [slots, H, d, dv].
extern "C" int b200_linear_scan(const void* q, const void* k, const void* v, int ldq, int ldk, int ldv, const float* gate, int ldg,
                                const float* decay, const float* beta, int ldb, float* state, float* out, int ldo,
                                const int* q_start, const int* slots, int entries, int tokens, int H, int Hqk, int d, int dv,
                                int act, int fixed_order, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (entries <= 0) return 0;
  if (H <= 0 || Hqk <= 0 || H % Hqk != 0 || d <= 0 || dv <= 0 || d > 256) return B200_ERR_BAD_SIZE;
  if ((gate == nullptr) == (decay == nullptr)) return B200_ERR_BAD_SIZE;
  ScanParams p{q, k, v, ldq, ldk, ldv, gate, ldg, decay, beta, ldb, state, out, ldo, q_start, slots, H, Hqk, d, dv, act, 1};
  p.rl = scan_row_lanes(entries, H, d, dv, tokens, fixed_order);
  const bool delta = beta != nullptr, gated = gate != nullptr;
  if (delta && gated) {
    B200_DISPATCH_DTYPE(dtype, T, return (launch_scan<T, true, true>(p, entries, stream)));
  } else if (!delta && !gated) {
    B200_DISPATCH_DTYPE(dtype, T, return (launch_scan<T, false, false>(p, entries, stream)));
  } else if (delta) {
    B200_DISPATCH_DTYPE(dtype, T, return (launch_scan<T, true, false>(p, entries, stream)));
  } else {
    B200_DISPATCH_DTYPE(dtype, T, return (launch_scan<T, false, true>(p, entries, stream)));
  }
  return 0;
}

extern "C" int b200_delta_prepare(const void* proj, int ld, int b_off, int a_off, int rank, const float* taps, int ntaps,
                                  const float* conv_state, const float* a_log, const float* dt_bias, const void* a_up,
                                  float* q, float* k, float* v, float* g, float* beta, const int* q_start, const int* slots,
                                  const int* token_entry, int n, int H, int G, int d, int dv, float unit_eps, float q_scale,
                                  int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G != 0 || d <= 0 || dv <= 0 || ntaps <= 0 || rank < 0) return B200_ERR_BAD_SIZE;
  DeltaPrepareParams p{proj, ld, b_off, a_off, rank, taps, ntaps, conv_state, a_log, dt_bias, a_up, q, k, v, g, beta,
                       q_start, slots, token_entry, H, G, d, dv, unit_eps, q_scale};
  const size_t smem = sizeof(float) * (static_cast<size_t>(2) * d + rank + static_cast<size_t>(rank) * d + (static_cast<size_t>(2) * d + dv) * ntaps);
  if (smem > 200 * 1024 || H > 65535) return B200_ERR_TOO_LARGE;
  // small batches: a CTA per token and head; prompt portions: eight tokens share a CTA's copy of the head's weights
  const int tokens_per_cta = n * H >= 8 * 2 * 148 ? 8 : 1;
  dim3 grid((n + tokens_per_cta - 1) / tokens_per_cta, H);
  static DeviceOnce once_f32, once_bf16;     // the opt-in to large shared memory is made once per device, for the largest sizes taken
  if (dtype == kF32) {
    if (int e = configure_once(once_f32, delta_prepare_kernel<float>, 200 * 1024)) return e;
    launch(delta_prepare_kernel<float>, grid, dim3(128), smem, stream, p, n, tokens_per_cta);
  } else if (dtype == kBF16) {
    if (int e = configure_once(once_bf16, delta_prepare_kernel<__nv_bfloat16>, 200 * 1024)) return e;
    launch(delta_prepare_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, p, n, tokens_per_cta);
  } else {
    return B200_ERR_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int b200_conv_state_update(const void* proj, int ld, float* conv_state, int C, int ntaps, const int* q_start,
                                      const int* slots, int entries, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (entries <= 0 || ntaps <= 1 || C <= 0) return 0;
  dim3 grid((C + 127) / 128, entries);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, launch(conv_state_update_kernel<T>, grid, dim3(128), 0, stream, static_cast<const T*>(proj), ld,
                                       conv_state, C, ntaps, q_start, slots));
  return launch_status();
}

extern "C" int b200_group_norm_gate(const float* x, int n, int width, int group, const float* w, float eps, const void* gate_in,
                                    int gate_ld, int rank, const void* gate_up, void* out, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || group <= 0 || width % group != 0 || rank < 0 || rank > 4096) return B200_ERR_BAD_SIZE;
  dim3 grid(n, width / group);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  const int threads = group >= 256 ? 256 : (group + 31) / 32 * 32;
  B200_DISPATCH_DTYPE(dtype, T, launch(group_norm_gate_kernel<T>, grid, dim3(threads), sizeof(float) * rank, stream, x, width, group,
                                       w, eps, static_cast<const T*>(gate_in), gate_ld, rank, static_cast<const T*>(gate_up),
                                       static_cast<T*>(out)));
  return launch_status();
}
