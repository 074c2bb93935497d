// Hyper-connections: the residual stream kept as S copies ("streams") per token.
//
// A sublayer q reads one mix of the streams and writes back into all of them:
//     u    = sum_s in[s] x_s                                  (what the sublayer's norm sees)
//     x_t <- sum_s mix[s, t] x_s + out[t] y                   (all streams at once from the old ones; y = sublayer(norm(u)))
// The streams of a token lie side by side in one float32 row [S * W].  As with the single stream, a sublayer's output
// stays pending until the next norm: hc_norm first applies the write of the sublayer before it (if any), stores the new
// streams, then forms u of its own sublayer and norms it (RMS norm with one number as gain), all in one pass over the
// row and in float32.  y may be a tensor or the unsummed partial results of a split-K product.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

template <typename T>
__global__ void hc_embedding_kernel(float* __restrict__ resid, const T* __restrict__ table, const int* __restrict__ ids,
                                    int hidden, int vocab, int streams, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* row = resid + (size_t)t * hidden * streams;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int c = threadIdx.x; c < hidden * streams; c += blockDim.x) row[c] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = to_f32(src[c]);
    for (int s = 0; s < streams; ++s) row[(size_t)s * hidden + c] = v;
  }
}

// One CTA per token.  write_mix [S, S] (from, to) and write_out [S]: the pending write (both null: nothing pending).
// read_in [S], gain (one number) and out: the read and norm that follow (out null: only the write is done).
template <typename T>
__global__ void __launch_bounds__(256)
hc_norm_kernel(float* __restrict__ resid, MaybePartial<T> y, const float* __restrict__ write_mix,
               const float* __restrict__ write_out, const float* __restrict__ read_in, const float* __restrict__ gain,
               T* __restrict__ out, int hidden, int streams, float eps) {
  extern __shared__ float u_s[];               // [hidden]
  __shared__ float red[32];
  __shared__ float mix_s[MAX_STREAMS * MAX_STREAMS], wout_s[MAX_STREAMS], win_s[MAX_STREAMS];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, S = streams;
  const bool pending = write_mix != nullptr;
  if (threadIdx.x < S * S && pending) mix_s[threadIdx.x] = write_mix[threadIdx.x];
  if (threadIdx.x < S) {
    wout_s[threadIdx.x] = pending ? write_out[threadIdx.x] : 0.f;
    win_s[threadIdx.x] = out ? read_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* row = resid + (size_t)t * hidden * S;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) x[s] = s < S ? row[(size_t)s * hidden + c] : 0.f;
    if (pending) {
      const float yv = y.at((size_t)t * hidden + c);
      float xn[MAX_STREAMS];
#pragma unroll
      for (int to = 0; to < MAX_STREAMS; ++to) {
        float a = 0.f;
        if (to < S) {
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) a = fmaf(mix_s[s * S + to], x[s], a);
          a = fmaf(wout_s[to], yv, a);
          row[(size_t)to * hidden + c] = a;
        }
        xn[to] = a;
      }
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s) x[s] = xn[s];
    }
    if (out) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) u = fmaf(win_s[s], x[s], u);
      u_s[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float r = 1.f / sqrtf(total / (float)hidden + eps) * gain[0];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[(size_t)t * hidden + c] = from_f32<T>(u_s[c] * r);
}

// The same with the stream count known at compile time and eight columns per thread: every access is 16 bytes wide
// (width a multiple of 8), the streams of a column group stay in registers between the write and the read.
template <typename T, int S>
__global__ void __launch_bounds__(256)
hc_norm_vec_kernel(float* __restrict__ resid, MaybePartial<T> y, const float* __restrict__ write_mix,
                   const float* __restrict__ write_out, const float* __restrict__ read_in, const float* __restrict__ gain,
                   T* __restrict__ out, int hidden, float eps) {
  extern __shared__ float u_s[];               // [hidden]
  __shared__ float red[32];
  __shared__ float mix_s[S * S], wout_s[S], win_s[S];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const bool pending = write_mix != nullptr;
  if (threadIdx.x < S * S && pending) mix_s[threadIdx.x] = write_mix[threadIdx.x];
  if (threadIdx.x < S) {
    wout_s[threadIdx.x] = pending ? write_out[threadIdx.x] : 0.f;
    win_s[threadIdx.x] = out ? read_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* row = resid + (size_t)t * hidden * S;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float x[S][8];
#pragma unroll
    for (int s = 0; s < S; ++s) Vec8<float>::load(row + (size_t)s * hidden + c, x[s]);
    if (pending) {
      float yv[8];
      y.at8((size_t)t * hidden + c, yv);
      float xn[S][8];
#pragma unroll
      for (int to = 0; to < S; ++to) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) a = fmaf(mix_s[s * S + to], x[s][i], a);
          xn[to][i] = fmaf(wout_s[to], yv[i], a);
        }
        Vec8<float>::store(row + (size_t)to * hidden + c, xn[to]);
      }
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int i = 0; i < 8; ++i) x[s][i] = xn[s][i];
    }
    if (out) {
      float u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) a = fmaf(win_s[s], x[s][i], a);
        u[i] = a;
        ss = fmaf(a, a, ss);
      }
      Vec8<float>::store(u_s + c, u);
    }
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float r = 1.f / sqrtf(total / (float)hidden + eps) * gain[0];
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float u[8];
    Vec8<float>::load(u_s + c, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) u[i] *= r;
    Vec8<T>::store(out + (size_t)t * hidden + c, u);
  }
}

__global__ void hc_gather_sum_kernel(float* __restrict__ out, const float* __restrict__ resid, const int* __restrict__ rows,
                                     int hidden, int streams) {
  pdl_launch_dependents();
  pdl_wait();
  const float* row = resid + (size_t)rows[blockIdx.x] * hidden * streams;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < streams; ++s) a += row[(size_t)s * hidden + c];
    out[(size_t)blockIdx.x * hidden + c] = a;
  }
}

// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * gain[0] for float32 rows (the rows before the head)
template <typename T>
__global__ void __launch_bounds__(256)
scalar_rmsnorm_rows_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ gain, int hidden, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = x + (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  const float total = block_sum(ss, red);
  const float r = 1.f / sqrtf(total / (float)hidden + eps) * gain[0];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[(size_t)blockIdx.x * hidden + c] = from_f32<T>(row[c] * r);
}

}  // namespace

// resid [n_tokens, streams * hidden] float32: every stream of token t = table[ids[t]]; an id outside the table sets *status
LLMK_API int llmk_hc_embedding(float* resid, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                               int streams, int dtype, int* status, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(streams >= 1 && streams <= MAX_STREAMS, "hc_embedding: %d streams (1 to %d)", streams, MAX_STREAMS);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(hc_embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, resid, (const T*)table, ids, hidden, vocab,
                  streams, status);
    LLMK_LAUNCH_CHECK("hc_embedding");
  });
}

// The pending write (write_mix, write_out and y; all absent: none), then the read and norm (read_in, gain, out; out null: none).
LLMK_API int llmk_hc_norm(float* resid, const void* y, const float* partials, int splits, long long split_stride,
                          const float* write_mix, const float* write_out, const float* read_in, const float* gain, void* out,
                          int n_tokens, int hidden, int streams, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(streams >= 1 && streams <= MAX_STREAMS, "hc_norm: %d streams (1 to %d)", streams, MAX_STREAMS);
  LLMK_REQUIRE(hidden > 0 && hidden <= 24576, "hc_norm: width %d (1 to 24576)", hidden);
  const bool pending = y != nullptr || partials != nullptr;
  LLMK_REQUIRE(pending == (write_mix != nullptr) && pending == (write_out != nullptr), "hc_norm: a pending term needs its weights");
  LLMK_REQUIRE(out == nullptr || (read_in != nullptr && gain != nullptr), "hc_norm: a norm needs its weights");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> yy{(const T*)y, partials, splits, split_stride};
    const size_t smem = (size_t)hidden * sizeof(float);
    const bool vec = hidden % 8 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)partials % 16 == 0 &&
                     split_stride % 4 == 0 && (uintptr_t)out % 16 == 0;
#define LLMK_HC_VEC(S)                                                                                                  \
  case S:                                                                                                               \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(hc_norm_vec_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    launch_kernel(hc_norm_vec_kernel<T, S>, dim3(n_tokens), dim3(256), smem, stream, resid, yy, write_mix, write_out,   \
                  read_in, gain, (T*)out, hidden, eps);                                                                 \
    LLMK_LAUNCH_CHECK("hc_norm");
    if (vec) {
      switch (streams) {
        LLMK_HC_VEC(1) LLMK_HC_VEC(2) LLMK_HC_VEC(3) LLMK_HC_VEC(4) LLMK_HC_VEC(5) LLMK_HC_VEC(6) LLMK_HC_VEC(7) LLMK_HC_VEC(8)
      }
    }
#undef LLMK_HC_VEC
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(hc_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(hc_norm_kernel<T>, dim3(n_tokens), dim3(256), smem, stream, resid, yy, write_mix, write_out, read_in, gain,
                  (T*)out, hidden, streams, eps);
    LLMK_LAUNCH_CHECK("hc_norm");
  });
}

// out[r] = sum over the streams of resid[rows[r]], float32
LLMK_API int llmk_hc_gather_sum(float* out, const float* resid, const int* rows, int n_rows, int hidden, int streams,
                                cudaStream_t stream) {
  if (n_rows == 0) return 0;
  launch_kernel(hc_gather_sum_kernel, dim3(n_rows), dim3(256), 0, stream, out, resid, rows, hidden, streams);
  LLMK_LAUNCH_CHECK("hc_gather_sum");
}

LLMK_API int llmk_scalar_rmsnorm_rows(void* out, const float* x, const float* gain, int n_rows, int hidden, float eps, int dtype,
                                      cudaStream_t stream) {
  if (n_rows == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(scalar_rmsnorm_rows_kernel<T>, dim3(n_rows), dim3(256), 0, stream, (T*)out, x, gain, hidden, eps);
    LLMK_LAUNCH_CHECK("scalar_rmsnorm_rows");
  });
}
