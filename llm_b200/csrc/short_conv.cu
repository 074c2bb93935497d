// A short causal convolution over time on each channel, with the request's last inputs kept as state.
//
//     y_t[c] = sum_{j < taps} w[c, j] x_(t - taps + 1 + j)[c]  (+ bias[c])          zeros before the sequence's start
// Options: out = x + y (the convolution as a side branch of its own input), and silu on the result.  The inputs of a
// request's last taps - 1 tokens live in its state slot (float32 [taps - 1, channels], oldest first, zero at admission),
// so a token's result is the same arithmetic whether its predecessors came in this step or in an earlier one.  The
// products and sums are float32; x is read and the result written in the element kind of the step.
//
// Two launches: the convolution (a thread per token and channel; it reads the old state), then the state's update
// (a thread per entry and channel, which walks the taps - 1 places in ascending order: place k takes either an input of
// this step or the old place k + n, which lies above every place written so far).  When every entry brings one token
// the convolution's thread is the only reader of its entry's places and moves them itself (place j - 1 takes what tap j
// read): one launch.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                  const float* __restrict__ w, const float* __restrict__ bias, float* state,
                  long long slot_stride, const int* __restrict__ state_slots, const int* __restrict__ token_entry,
                  const int* __restrict__ cu_tokens, int channels, int taps, int residual, int act, int single) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int e = token_entry[t];
  const int start = cu_tokens[e];
  float* st = state + (size_t)state_slots[e] * slot_stride;
  float y = bias ? bias[c] : 0.f;
  float self = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = t - (taps - 1) + j;
    float v;
    if (src >= start) v = to_f32(x[(size_t)src * x_stride + c]);
    else v = st[(size_t)(taps - 1 + src - start) * channels + c];      // place k holds the input at start - (taps - 1) + k
    if (j == taps - 1) self = v;
    if (single && j >= 1) st[(size_t)(j - 1) * channels + c] = v;
    y = fmaf(w[(size_t)j * channels + c], v, y);
  }
  if (residual) y += self;
  if (act) y = y / (1.f + expf(-y));
  out[(size_t)t * out_stride + c] = from_f32<T>(y);
}

// The same for eight channels a thread (16-byte accesses; channels a multiple of 8, at most TAPS taps) and `run` consecutive
// tokens a thread, with the thread's weights in registers.  A token's rows are read again for the next token; they come
// from the first-level cache.  The sums run over the taps in the same order as above.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
short_conv_vec_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                      const float* __restrict__ w, const float* __restrict__ bias, float* state,
                      long long slot_stride, const int* __restrict__ state_slots, const int* __restrict__ token_entry,
                      const int* __restrict__ cu_tokens, int n_tokens, int channels, int taps, int residual, int act, int run,
                      int single) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= channels) return;
  float wr[TAPS][8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = bias ? bias[c + i] : 0.f;
#pragma unroll
  for (int j = 0; j < TAPS; ++j) {
    if (j < taps) Vec8<float>::load(w + (size_t)j * channels + c, wr[j]);
  }
  const int t_end = min(n_tokens, (int)(blockIdx.x + 1) * run);
  for (int t = blockIdx.x * run; t < t_end; ++t) {
    const int e = token_entry[t];
    const int start = cu_tokens[e];
    float* st = state + (size_t)state_slots[e] * slot_stride;
    float y[8], v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = b[i];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      if (j >= taps) break;
      const int src = t - (taps - 1) + j;
      if (src >= start) Vec8<T>::load(x + (size_t)src * x_stride + c, v);
      else Vec8<float>::load(st + (size_t)(taps - 1 + src - start) * channels + c, v);
      if (single && j >= 1) Vec8<float>::store(st + (size_t)(j - 1) * channels + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = fmaf(wr[j][i], v[i], y[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {                    // v holds the token's own input (the last tap)
      if (residual) y[i] += v[i];
      if (act) y[i] = y[i] / (1.f + expf(-y[i]));
    }
    Vec8<T>::store(out + (size_t)t * out_stride + c, y);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const T* __restrict__ x, long long x_stride, float* __restrict__ state, long long slot_stride,
                        const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int start = cu_tokens[e], n = cu_tokens[e + 1] - start;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[e] * slot_stride;
  for (int k = 0; k < taps - 1; ++k) {
    const int p = n - (taps - 1) + k;                  // the place's token, counted from the entry's first
    const float v = p >= 0 ? to_f32(x[(size_t)(start + p) * x_stride + c]) : st[(size_t)(k + n) * channels + c];
    st[(size_t)k * channels + c] = v;
  }
}

}  // namespace

// x, out [n_tokens, stride] (out may not be x); w float32 [taps, channels] (a row per tap, oldest first); bias float32 [channels] or null;
// state float32, slot s at state + s * slot_stride, [taps - 1, channels].
LLMK_API int llmk_short_conv(void* out, long long out_stride, const void* x, long long x_stride, const float* w, const float* bias,
                             float* state, long long slot_stride, const int* state_slots, const int* token_entry,
                             const int* cu_tokens, int n_tokens, int n_entries, int channels, int taps, int residual, int act,
                             int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "short_conv: %d taps (1 to %d)", taps, MAX_TAPS);
  LLMK_REQUIRE(out != x, "short_conv: the result needs a place of its own");
  LLMK_REQUIRE(slot_stride >= (long long)(taps - 1) * channels, "short_conv: a state slot of %lld numbers is too small", slot_stride);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    const unsigned bx = (unsigned)((channels + 255) / 256);
    constexpr int per16 = 16 / (int)sizeof(T);
    const bool vec = channels % 8 == 0 && taps <= 8 && (uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0 && out_stride % per16 == 0 &&
                     x_stride % per16 == 0 && (uintptr_t)state % 16 == 0 && slot_stride % 4 == 0 && (uintptr_t)w % 16 == 0;
    cudaError_t err;
    const int single = n_tokens == n_entries;                  // every entry brings one token: the convolution moves the state
    if (vec) {
      const int run = n_tokens >= 4096 ? 8 : n_tokens >= 512 ? 4 : 1;      // long steps: a thread keeps its weights for some tokens
      const dim3 grid((unsigned)((n_tokens + run - 1) / run), (unsigned)((channels / 8 + 127) / 128));
      if (taps <= 4)
        err = launch_kernel(short_conv_vec_kernel<T, 4>, grid, dim3(128), 0, stream, (T*)out, out_stride, (const T*)x, x_stride, w, bias,
                            state, slot_stride, state_slots, token_entry, cu_tokens, n_tokens, channels, taps, residual,
                            act, run, single);
      else
        err = launch_kernel(short_conv_vec_kernel<T, 8>, grid, dim3(128), 0, stream, (T*)out, out_stride, (const T*)x, x_stride, w, bias,
                            state, slot_stride, state_slots, token_entry, cu_tokens, n_tokens, channels, taps, residual,
                            act, run, single);
    } else {
      err = launch_kernel(short_conv_kernel<T>, dim3(n_tokens, bx), dim3(256), 0, stream, (T*)out, out_stride, (const T*)x,
                          x_stride, w, bias, state, slot_stride, state_slots, token_entry, cu_tokens,
                          channels, taps, residual, act, single);
    }
    if (err == cudaSuccess && taps > 1 && !single)
      launch_kernel(short_conv_state_kernel<T>, dim3(bx, n_entries), dim3(256), 0, stream, (const T*)x, x_stride, state,
                    slot_stride, state_slots, cu_tokens, channels, taps);
    LLMK_LAUNCH_CHECK("short_conv");
  });
}
