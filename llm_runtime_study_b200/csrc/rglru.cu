// A gated linear recurrence per channel behind a short causal convolution (the recurrent block of Griffin:
// De, Smith, Fernando et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient
// Language Models").  The state, the gates, the decay and its logarithm are float32.
//
//   u_t   = conv(x)_t + conv_bias                    (taps over time, the last tap is the current token's)
//   r, i  = sigmoid(gate logits)                     (formed by a block-diagonal product outside these kernels)
//   log a = -c r softplus(lam),  a = exp(log a)
//   S_t   = a S_(t-1) + sqrt(1 - a^2) i u_t          (S = 0 before the first token)
//   out_t = S_t * gelu_tanh(y_t)
#include "common.cuh"

namespace b200 {

// One thread per (token, channel).  x is the first `width` columns of the stacked projection rows; inputs before the
// step come from the slot's kept rows [slots, taps-1, width] (oldest first).
template <typename T>
__global__ void __launch_bounds__(256)
conv_taps_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ taps, const float* __restrict__ bias, int ntaps,
                 const float* __restrict__ conv_state, const int* __restrict__ q_start, const int* __restrict__ slots,
                 const int* __restrict__ token_entry, T* __restrict__ u, int width) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int entry = token_entry[token];
  const int first = q_start[entry];
  const int local = token - first;
  const float* kept = conv_state + static_cast<size_t>(slots[entry]) * (ntaps - 1) * width;
  float acc = bias[c];
  for (int j = 0; j < ntaps; ++j) {
    const int back = ntaps - 1 - j;          // tap j multiplies the input `back` tokens ago
    const int at = local - back;
    const float x = at >= 0 ? to_float(proj[static_cast<size_t>(first + at) * ld + c])
                            : kept[static_cast<size_t>(ntaps - 1 + at) * width + c];
    acc = fmaf(taps[static_cast<size_t>(c) * ntaps + j], x, acc);
  }
  u[static_cast<size_t>(token) * width + c] = from_float<T>(acc);
}

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The gates' arithmetic for every (token, channel) at once, all of it independent of the state: a = exp(-c r softplus(lam)),
// b = sqrt(1 - a^2) i u, and gelu_tanh(y) in the activation type.  gates: float32 [n, blocks, 2 * bw] (r logits, then i
// logits, of the block's channels); y: column y_off + c of the projection rows.
template <typename T>
__global__ void __launch_bounds__(256)
recurrence_inputs_kernel(const float* __restrict__ gates, const T* __restrict__ u, const T* __restrict__ proj, int ld, int y_off,
                         const float* __restrict__ lam, float decay_scale, float* __restrict__ a_out, float* __restrict__ b_out,
                         T* __restrict__ y_out, int width, int bw) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const float lm = lam[c];
  const float sp = lm > 20.f ? lm : log1pf(expf(lm));
  const int block = c / bw, o = c - block * bw;
  const float* g = gates + (static_cast<size_t>(t) * (width / bw) + block) * 2 * bw;
  const float r = 1.f / (1.f + expf(-g[o]));
  const float i = 1.f / (1.f + expf(-g[bw + o]));
  const float log_a = -decay_scale * r * sp;
  const size_t at = static_cast<size_t>(t) * width + c;
  a_out[at] = expf(log_a);
  b_out[at] = sqrtf(-expm1f(2.f * log_a)) * i * to_float(u[at]);
  y_out[at] = from_float<T>(gelu_tanh(to_float(proj[static_cast<size_t>(t) * ld + y_off + c])));
}

// One thread per (entry, channel) walks the entry's tokens in order: S <- a S + b, out = S * y.  Only the multiply-adds form
// a chain; the loads of sixteen tokens are in flight together.  state [slots, width]; y is read and the result written in place.
template <typename T>
__global__ void __launch_bounds__(128)
gated_recurrence_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ y, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ slots, int width) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int first = q_start[entry], last = q_start[entry + 1];
  float* st = state + static_cast<size_t>(slots[entry]) * width + c;
  float S = *st;
  constexpr int U = 16;
  int t0 = first;
  for (; t0 + U <= last; t0 += U) {
    float av[U], bv[U], yv[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const size_t at = static_cast<size_t>(t0 + j) * width + c;
      av[j] = a[at];
      bv[j] = b[at];
      yv[j] = to_float(y[at]);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      S = fmaf(av[j], S, bv[j]);
      y[static_cast<size_t>(t0 + j) * width + c] = from_float<T>(S * yv[j]);
    }
  }
  for (; t0 < last; ++t0) {
    const size_t at = static_cast<size_t>(t0) * width + c;
    S = fmaf(a[at], S, b[at]);
    y[at] = from_float<T>(S * to_float(y[at]));
  }
  *st = S;
}

}  // namespace b200

extern "C" int b200_conv_taps(const void* proj, int ld, const float* taps, const float* bias, int ntaps, const float* conv_state,
                              const int* q_start, const int* slots, const int* token_entry, void* u, int n, int width, int dtype,
                              cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (width <= 0 || ntaps <= 0 || ld < width || (ntaps > 1 && conv_state == nullptr)) return B200_ERR_BAD_SIZE;
  dim3 grid(n, (width + 255) / 256);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, launch(conv_taps_kernel<T>, grid, dim3(256), 0, stream, static_cast<const T*>(proj), ld, taps, bias,
                                       ntaps, conv_state, q_start, slots, token_entry, static_cast<T*>(u), width));
  return launch_status();
}

// gates float32 [n, width / bw, 2 * bw]; u [n, width] and proj rows in the activation type; a_scratch, b_scratch float32 [n, width];
// out [n, width] in the activation type.
extern "C" int b200_gated_recurrence(const float* gates, const void* u, const void* proj, int ld, int y_off, const float* lam,
                                     float decay_scale, float* state, const int* q_start, const int* slots, void* out,
                                     float* a_scratch, float* b_scratch, int n, int entries, int width, int bw, int dtype,
                                     cudaStream_t stream) {
  using namespace b200;
  if (entries <= 0 || n <= 0) return 0;
  if (width <= 0 || bw <= 0 || width % bw != 0 || ld < y_off + width) return B200_ERR_BAD_SIZE;
  dim3 wide(n, (width + 255) / 256), grid((width + 127) / 128, entries);
  if (grid.y > 65535 || wide.y > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, {
    launch(recurrence_inputs_kernel<T>, wide, dim3(256), 0, stream, gates, static_cast<const T*>(u), static_cast<const T*>(proj), ld,
           y_off, lam, decay_scale, a_scratch, b_scratch, static_cast<T*>(out), width, bw);
    launch(gated_recurrence_kernel<T>, grid, dim3(128), 0, stream, a_scratch, b_scratch, static_cast<T*>(out), state, q_start, slots,
           width);
  });
  return launch_status();
}
