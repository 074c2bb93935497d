// Row-wise kernels: embedding gather, residual add fused with RMSNorm, row gather
// for the LM head, SiLU(gate) * up.  The residual stream is float32 in every mode;
// sums, the reciprocal root and the scaling are float32 as well.  An input that comes
// from a split-K product may be given as its float32 partial results, which are summed
// here in a fixed order instead of by a kernel of their own.
#include "common.cuh"

// ---- embedding --------------------------------------------------------------
// resid[t, :] = table[ids[t], :]   (the reference copies rows without scaling,
// kernel/embedding/TokenEmbedding.h:12-17).  An id outside the table sets *status.
template <typename T>
__global__ void embedding_kernel(float* __restrict__ resid, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab,
                                 int* __restrict__ status, float scale) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) resid[(size_t)t * hidden + c] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) resid[(size_t)t * hidden + c] = to_f32(row[c]) * scale;
}

// scale: every row is multiplied by it in float32 on its way into the stream (1 = the plain copy).
LLMK_API int llmk_embedding_scaled(float* resid, const void* table, const int* ids, int n_tokens, int hidden,
                                   int vocab, int dtype, int* status, float scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, resid, (const T*)table, ids, hidden, vocab, status,
                  scale);
    LLMK_LAUNCH_CHECK("embedding");
  });
}

LLMK_API int llmk_embedding(float* resid, const void* table, const int* ids, int n_tokens, int hidden,
                            int vocab, int dtype, int* status, cudaStream_t stream) {
  return llmk_embedding_scaled(resid, table, ids, n_tokens, hidden, vocab, dtype, status, 1.f, stream);
}

// ---- residual add + RMSNorm -------------------------------------------------
// resid += delta (if delta); out = resid * rsqrt(mean(resid^2) + eps) * gamma.
// The reference runs the add and the norm as two kernels (kernel/residual/Residual.h:17-19,
// kernel/LayerNorm/RMSNorm.h:13-30,40-42); here they share one pass over the row.
template <typename T, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, MaybePartial<T> delta,
                                   const float* __restrict__ gamma, T* __restrict__ out, int hidden,
                                   float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  const bool has_delta = delta.present();
  float ss = 0.f;
  if (VEC) {
    // eight elements per thread and pass; a row of up to 8 * blockDim stays in registers
    float keep[8];
    const bool single = hidden <= 8 * (int)blockDim.x;
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      float v[8];
      Vec8<float>::load(resid + base + c, v);
      if (has_delta) {
        float d[8];
        delta.at8(base + c, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += d[i];
        Vec8<float>::store(resid + base + c, v);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) { ss += v[i] * v[i]; keep[i] = v[i]; }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    if (out) {
      for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
        float v[8], g[8];
        if (single) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = keep[i];
        } else {
          Vec8<float>::load(resid + base + c, v);
        }
        Vec8<float>::load(gamma + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * g[i];
        Vec8<T>::store(out + base + c, v);
      }
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[base + c];
    if (has_delta) {
      v += delta.at(base + c);
      resid[base + c] = v;
    }
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (out) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
      out[base + c] = from_f32<T>(resid[base + c] * rstd * gamma[c]);
  }
}

// delta: [rows, hidden] of the element kind, or null; partials: [splits][rows][hidden] float32
// (split_stride elements apart), or null.  At most one of the two is given.
LLMK_API int llmk_add_rmsnorm(float* resid, const void* delta, const float* partials, int splits,
                              long long split_stride, const float* gamma, void* out, int rows, int hidden,
                              float eps, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "add_rmsnorm: give delta or partials, not both");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    const bool vec = hidden % 8 == 0 && d.vector_ok() && (uintptr_t)resid % 16 == 0 && (uintptr_t)gamma % 16 == 0 &&
                     (uintptr_t)out % 16 == 0;
    if (vec)
      launch_kernel(add_rmsnorm_kernel<T, true>, dim3(rows), dim3(256), 0, stream, resid, d, gamma, (T*)out, hidden, eps);
    else
      launch_kernel(add_rmsnorm_kernel<T, false>, dim3(rows), dim3(256), 0, stream, resid, d, gamma, (T*)out, hidden, eps);
    LLMK_LAUNCH_CHECK("add_rmsnorm");
  });
}

// ---- gather of the rows whose logits are wanted -----------------------------
// out[r, :] = resid[rows[r], :] (+ delta[rows[r], :]).  The reference runs its LM head
// on every row (model/modules/Linear.h:25); gathering first leaves only wanted rows.
template <typename T>
__global__ void gather_rows_kernel(float* __restrict__ out, const float* __restrict__ resid,
                                   MaybePartial<T> delta, const int* __restrict__ rows, int hidden) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const size_t src = (size_t)rows[blockIdx.x] * hidden, dst = (size_t)blockIdx.x * hidden;
  const bool has_delta = delta.present();
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[src + c];
    if (has_delta) v += delta.at(src + c);
    out[dst + c] = v;
  }
}

LLMK_API int llmk_gather_rows(float* out, const float* resid, const void* delta, const float* partials,
                              int splits, long long split_stride, const int* rows, int n_rows, int hidden,
                              int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "gather_rows: give delta or partials, not both");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    launch_kernel(gather_rows_kernel<T>, dim3(n_rows), dim3(256), 0, stream, out, resid, d, rows, hidden);
    LLMK_LAUNCH_CHECK("gather_rows");
  });
}

// out[i] = in[i] rounded to the element type: float32 rows handed to a product without a norm
// between (a head that takes the stream as it is).
template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ in, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(in[i]);
}

LLMK_API int llmk_cast_rows(void* out, const float* in, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  size_t blocks = ((size_t)n + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 8) blocks = (size_t)llmk_sm_count() * 8;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(cast_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, (size_t)n);
    LLMK_LAUNCH_CHECK("cast_rows");
  });
}

// x[r, c] += bias[c] (float32 sum, rounded once): the bias of a projection whose product is
// already summed.  The reference adds it in its products' epilogues (kernel/Gemm/QKVGemm.h:27-45,
// model/modules/Linear.h:12-34).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long long stride, const float* __restrict__ bias, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols;
    const int c = (int)(i - r * cols);
    T* p = x + r * stride + c;
    *p = from_f32<T>(to_f32(*p) + bias[c]);
  }
}

LLMK_API int llmk_add_bias(void* x, long long stride, const float* bias, int rows, int cols, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  size_t blocks = ((size_t)rows * cols + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 16) blocks = (size_t)llmk_sm_count() * 16;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(add_bias_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)x, stride, bias, rows, cols);
    LLMK_LAUNCH_CHECK("add_bias");
  });
}

// ---- SiLU(gate) * up --------------------------------------------------------
// in [rows, 2*inter]: gate in the first half of a row, up in the second.
// act = g / (1 + exp(-g)) * u in float32 (kernel/activation/SwiGLU.h:31-33).
template <typename T, bool VEC>
__global__ void silu_mul_kernel(T* __restrict__ out, MaybePartial<T> in, int inter, size_t total, int relu) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  if (VEC) {
    const unsigned per_row = inter / 8;
    const size_t n_vec = total / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
      const size_t r = i / per_row;
      const unsigned c = (unsigned)(i - r * per_row) * 8;
      float g[8], u[8];
      in.at8(r * 2 * inter + c, g);
      in.at8(r * 2 * inter + inter + c, u);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = (relu ? fmaxf(g[k], 0.f) : g[k] / (1.0f + expf(-g[k]))) * u[k];
      Vec8<T>::store(out + r * inter + c, g);
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i % inter;
    const float g = in.at(r * 2 * inter + c);
    const float u = in.at(r * 2 * inter + inter + c);
    out[i] = from_f32<T>((relu ? fmaxf(g, 0.f) : g / (1.0f + expf(-g))) * u);
  }
}

// act 0: silu(gate) * up; 1: relu(gate) * up.
LLMK_API int llmk_glu_mul(void* out, const void* gate_up, const float* partials, int splits,
                          long long split_stride, int rows, int inter, int dtype, int act, cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  LLMK_REQUIRE((gate_up != nullptr) != (partials != nullptr), "glu_mul: give gate_up or partials");
  LLMK_REQUIRE(act == 0 || act == 1, "glu_mul: activation %d is not silu (0) or relu (1)", act);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> in{(const T*)gate_up, partials, splits, split_stride};
    const bool vec = inter % 8 == 0 && in.vector_ok() && (uintptr_t)out % 16 == 0;
    size_t blocks = ((vec ? total / 8 : total) + 255) / 256;
    if (blocks > (size_t)llmk_sm_count() * 32) blocks = (size_t)llmk_sm_count() * 32;
    if (vec)
      launch_kernel(silu_mul_kernel<T, true>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, inter, total, act);
    else
      launch_kernel(silu_mul_kernel<T, false>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, in, inter, total, act);
    LLMK_LAUNCH_CHECK("silu_mul");
  });
}

LLMK_API int llmk_silu_mul(void* out, const void* gate_up, const float* partials, int splits,
                           long long split_stride, int rows, int inter, int dtype, cudaStream_t stream) {
  return llmk_glu_mul(out, gate_up, partials, splits, split_stride, rows, inter, dtype, 0, stream);
}

// ---- residual add + Dynamic Tanh ----------------------------------------------
// resid += delta (if delta); out = tanh(alpha * resid) * w + b.  A norm without a mean or a
// variance: every element stands alone, so the kernel is a plain sweep over rows * hidden.
template <typename T>
__global__ void add_dyt_kernel(float* __restrict__ resid, MaybePartial<T> delta, const float* __restrict__ w,
                               const float* __restrict__ b, float alpha, T* __restrict__ out, int hidden, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const bool has_delta = delta.present();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = resid[i];
    if (has_delta) {
      v += delta.at(i);
      resid[i] = v;
    }
    if (out) {
      const int c = (int)(i % hidden);
      out[i] = from_f32<T>(fmaf(tanhf(alpha * v), w[c], b[c]));
    }
  }
}

// eight elements per thread (16-byte accesses) where the row length and the pointers allow it
template <typename T>
__global__ void add_dyt8_kernel(float* __restrict__ resid, MaybePartial<T> delta, const float* __restrict__ w,
                                const float* __restrict__ b, float alpha, T* __restrict__ out, int hidden, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  const bool has_delta = delta.present();
  const int per_row = hidden / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t at = i * 8;
    const int c = (int)(i % per_row) * 8;
    float v[8];
    Vec8<float>::load(resid + at, v);
    if (has_delta) {
      float d[8];
      delta.at8(at, d);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += d[k];
      Vec8<float>::store(resid + at, v);
    }
    if (out) {
      float g[8], o[8];
      Vec8<float>::load(w + c, g);
      Vec8<float>::load(b + c, o);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = fmaf(tanhf(alpha * v[k]), g[k], o[k]);
      Vec8<T>::store(out + at, v);
    }
  }
}

LLMK_API int llmk_add_dyt(float* resid, const void* delta, const float* partials, int splits, long long split_stride,
                          const float* w, const float* b, float alpha, void* out, int rows, int hidden, int dtype,
                          cudaStream_t stream) {
  if (rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "add_dyt: give delta or partials, not both");
  const size_t total = (size_t)rows * hidden;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 16) blocks = (size_t)llmk_sm_count() * 16;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    const bool vec = hidden % 8 == 0 && d.vector_ok() && (uintptr_t)resid % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                     (uintptr_t)b % 16 == 0 && (uintptr_t)out % 16 == 0;
    if (vec) {
      size_t b8 = (total / 8 + 255) / 256;
      if (b8 > (size_t)llmk_sm_count() * 16) b8 = (size_t)llmk_sm_count() * 16;
      launch_kernel(add_dyt8_kernel<T>, dim3((unsigned)b8), dim3(256), 0, stream, resid, d, w, b, alpha, (T*)out, hidden, total / 8);
    } else {
      launch_kernel(add_dyt_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, resid, d, w, b, alpha, (T*)out, hidden, total);
    }
    LLMK_LAUNCH_CHECK("add_dyt");
  });
}

// ---- element-wise activations -------------------------------------------------
// out = act(in), float32 arithmetic; in a tensor or the partial results of a split-K product.
// kind 0: relu(z)^2; 1: gelu with erf; 2: gelu with tanh; 3: z * sigmoid(z); 4: tanh(z).
enum : int { LLMK_ACT_RELU2 = 0, LLMK_ACT_GELU_ERF = 1, LLMK_ACT_GELU_TANH = 2, LLMK_ACT_SILU = 3, LLMK_ACT_TANH = 4 };

__device__ __forceinline__ float apply_act(float z, int kind) {
  switch (kind) {
    case LLMK_ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    case LLMK_ACT_GELU_ERF: return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
    case LLMK_ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    case LLMK_ACT_TANH: return tanhf(z);
    default: return z / (1.f + expf(-z));
  }
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ out, MaybePartial<T> in, int kind, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(apply_act(in.at(i), kind));
}

template <typename T>
__global__ void act_rows8_kernel(T* __restrict__ out, MaybePartial<T> in, int kind, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8];
    in.at8(i * 8, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = apply_act(v[k], kind);
    Vec8<T>::store(out + i * 8, v);
  }
}

LLMK_API int llmk_act_rows(void* out, const void* in, const float* partials, int splits, long long split_stride,
                           long long total, int kind, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  LLMK_REQUIRE((in != nullptr) != (partials != nullptr), "act_rows: give in or partials");
  LLMK_REQUIRE(kind >= 0 && kind <= 4, "act_rows: unknown activation %d", kind);
  size_t blocks = ((size_t)total + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 32) blocks = (size_t)llmk_sm_count() * 32;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> x{(const T*)in, partials, splits, split_stride};
    if (total % 8 == 0 && x.vector_ok() && (uintptr_t)out % 16 == 0) {
      size_t b8 = ((size_t)total / 8 + 255) / 256;
      if (b8 > (size_t)llmk_sm_count() * 32) b8 = (size_t)llmk_sm_count() * 32;
      launch_kernel(act_rows8_kernel<T>, dim3((unsigned)b8), dim3(256), 0, stream, (T*)out, x, kind, (size_t)total / 8);
    } else {
      launch_kernel(act_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, x, kind, (size_t)total);
    }
    LLMK_LAUNCH_CHECK("act_rows");
  });
}

// ---- LayerNorm around a sublayer ------------------------------------------------
// A block that norms a sublayer's output before it joins the residual, and norms the residual
// before the next sublayer, needs per row
//     resid += mult * ln(delta; post)        (post null: resid += mult * delta)
//     out    = ln(resid; pre)                (out null: nothing more)
// with ln(x; w) = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w: a weight, no bias, the
// variance taken from the deviations (two passes over the row in shared memory).  Both halves are
// optional, all arithmetic is float32, and a row is read from memory once.
template <typename T>
__global__ void __launch_bounds__(256)
add_layernorm_kernel(float* __restrict__ resid, MaybePartial<T> delta, const float* __restrict__ post, float mult,
                     const float* __restrict__ pre, T* __restrict__ out, int hidden, float eps) {
  extern __shared__ float row_s[];
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  const float inv_n = 1.f / (float)hidden;
  if (delta.present()) {
    float s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = delta.at(base + c);
      row_s[c] = v;
      s += v;
    }
    float mean = 0.f, rstd = 1.f;
    if (post) {
      mean = block_sum(s, scratch) * inv_n;
      float q = 0.f;
      for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float d = row_s[c] - mean;
        q += d * d;
      }
      rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float y = post ? (row_s[c] - mean) * rstd * post[c] : row_s[c];
      const float r = fmaf(mult, y, resid[base + c]);
      resid[base + c] = r;
      row_s[c] = r;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) row_s[c] = resid[base + c];
  }
  if (!out) return;
  float s = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) s += row_s[c];
  const float mean = block_sum(s, scratch) * inv_n;
  float q = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float d = row_s[c] - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    out[base + c] = from_f32<T>((row_s[c] - mean) * rstd * pre[c]);
}

// The same for rows of up to NV * 2048 elements on the 8-grid: the row stays in registers (NV vectors of eight per
// thread), every access is 16 bytes wide, and the statistics are the same two passes (mean, then squared deviations).
template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(float* __restrict__ resid, MaybePartial<T> delta, const float* __restrict__ post, float mult,
                         const float* __restrict__ pre, T* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  const float inv_n = 1.f / (float)hidden;
  float r[NV][8];
  if (delta.present()) {
    float y[NV][8];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 256 + threadIdx.x) * 8;
      if (c < hidden) {
        delta.at8(base + c, y[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += y[v][i];
      }
    }
    float mean = 0.f, rstd = 1.f;
    if (post) {
      mean = block_sum(s, scratch) * inv_n;
      float q = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if ((v * 256 + threadIdx.x) * 8 < hidden) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = y[v][i] - mean; q += d * d; }
        }
      }
      rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 256 + threadIdx.x) * 8;
      if (c < hidden) {
        Vec8<float>::load(resid + base + c, r[v]);
        if (post) {
          float w[8];
          Vec8<float>::load(post + c, w);
#pragma unroll
          for (int i = 0; i < 8; ++i) r[v][i] = fmaf(mult, (y[v][i] - mean) * rstd * w[i], r[v][i]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) r[v][i] = fmaf(mult, y[v][i], r[v][i]);
        }
        Vec8<float>::store(resid + base + c, r[v]);
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * 256 + threadIdx.x) * 8;
      if (c < hidden) Vec8<float>::load(resid + base + c, r[v]);
    }
  }
  if (!out) return;
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if ((v * 256 + threadIdx.x) * 8 < hidden) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s += r[v][i];
    }
  }
  const float mean = block_sum(s, scratch) * inv_n;
  float q = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if ((v * 256 + threadIdx.x) * 8 < hidden) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float d = r[v][i] - mean; q += d * d; }
    }
  }
  const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = (v * 256 + threadIdx.x) * 8;
    if (c < hidden) {
      float w[8], o[8];
      Vec8<float>::load(pre + c, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (r[v][i] - mean) * rstd * w[i];
      Vec8<T>::store(out + base + c, o);
    }
  }
}

// delta: [rows, hidden] of the element kind, or float32 partial results, or neither; post, pre: float32
// [hidden] or null; out: [rows, hidden] of the element kind or null (then pre is not read).
LLMK_API int llmk_add_layernorm(float* resid, const void* delta, const float* partials, int splits, long long split_stride,
                                const float* post, float mult, const float* pre, void* out, int rows, int hidden, float eps,
                                int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  LLMK_REQUIRE(!(delta && partials), "add_layernorm: give delta or partials, not both");
  LLMK_REQUIRE(out == nullptr || pre != nullptr, "add_layernorm: an output needs its weight");
  const size_t smem = (size_t)hidden * sizeof(float);
  LLMK_REQUIRE(smem <= 200 * 1024, "add_layernorm: rows of %d elements exceed the shared memory", hidden);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> d{(const T*)delta, partials, splits, split_stride};
    const bool vec = hidden % 8 == 0 && hidden <= 8192 && d.vector_ok() && (uintptr_t)resid % 16 == 0 && (uintptr_t)post % 16 == 0 &&
                     (uintptr_t)pre % 16 == 0 && (uintptr_t)out % 16 == 0;
    if (vec && hidden <= 2048)
      launch_kernel(add_layernorm_vec_kernel<T, 1>, dim3(rows), dim3(256), 0, stream, resid, d, post, mult, pre, (T*)out, hidden, eps);
    else if (vec && hidden <= 4096)
      launch_kernel(add_layernorm_vec_kernel<T, 2>, dim3(rows), dim3(256), 0, stream, resid, d, post, mult, pre, (T*)out, hidden, eps);
    else if (vec)
      launch_kernel(add_layernorm_vec_kernel<T, 4>, dim3(rows), dim3(256), 0, stream, resid, d, post, mult, pre, (T*)out, hidden, eps);
    else {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(add_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      launch_kernel(add_layernorm_kernel<T>, dim3(rows), dim3(256), smem, stream, resid, d, post, mult, pre, (T*)out, hidden, eps);
    }
    LLMK_LAUNCH_CHECK("add_layernorm");
  });
}

// ---- soft cap ---------------------------------------------------------------------
// x = cap * tanh(x / cap), float32 in place: bounds logits to (-cap, cap) and leaves small ones alone.
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv_cap);
}

LLMK_API int llmk_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n == 0) return 0;
  LLMK_REQUIRE(cap > 0.f, "softcap: the cap must be positive");
  size_t blocks = ((size_t)n + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 16) blocks = (size_t)llmk_sm_count() * 16;
  launch_kernel(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, (size_t)n, cap, 1.f / cap);
  LLMK_LAUNCH_CHECK("softcap");
}

// ---- the stream beside the embedding ----------------------------------------------
// out[t] = [ resid[t] rounded to the element kind ; table[ids[t]] ]: the input of a product that mixes
// the stream with the embedding of the same token (width 2 * hidden).
template <typename T>
__global__ void concat_embedding_kernel(T* __restrict__ out, const float* __restrict__ resid, const T* __restrict__ table,
                                        const int* __restrict__ ids, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;            // the embedding kernel has reported a bad id already
  T* dst = out + (size_t)t * 2 * hidden;
  const T* row = table + (size_t)(ok ? id : 0) * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    dst[c] = from_f32<T>(resid[(size_t)t * hidden + c]);
    dst[hidden + c] = ok ? row[c] : from_f32<T>(0.f);
  }
}

LLMK_API int llmk_concat_embedding(void* out, const float* resid, const void* table, const int* ids, int n_tokens,
                                   int hidden, int vocab, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(concat_embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)out, resid, (const T*)table, ids,
                  hidden, vocab);
    LLMK_LAUNCH_CHECK("concat_embedding");
  });
}

// ---- RMS norm per head, gated -------------------------------------------------------
// out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * w[:] * silu(gate[t, h, :]): the output stage
// of a linear-attention mixer (x float32, one weight vector shared by the heads).  A warp per (t, h).
template <typename T>
__global__ void __launch_bounds__(128)
head_rmsnorm_gate_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                         const T* __restrict__ gate, long long gate_stride, long long items, int heads, int vdim, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = (int)(item % heads);
  const float* row = x + (size_t)item * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss += row[c] * row[c];
  const float rstd = rsqrtf(warp_sum(ss) / (float)vdim + eps);
  const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
  for (int c = lane; c < vdim; c += 32) {
    float y = row[c] * rstd * w[c];
    if (g) {
      const float z = to_f32(g[c]);
      y *= z / (1.f + expf(-z));
    }
    out[(size_t)item * vdim + c] = from_f32<T>(y);
  }
}

LLMK_API int llmk_head_rmsnorm_gate(void* out, const float* x, const float* w, const void* gate, long long gate_stride,
                                    int n_tokens, int heads, int vdim, float eps, int dtype, cudaStream_t stream) {
  const long long items = (long long)n_tokens * heads;
  if (items == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(head_rmsnorm_gate_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (T*)out, x, w,
                  (const T*)gate, gate_stride, items, heads, vdim, eps);
    LLMK_LAUNCH_CHECK("head_rmsnorm_gate");
  });
}

// ---- two attention maps combined per head ---------------------------------------------
// Differential attention's output stage.  a holds 2 * heads attention outputs of vdim per token, ordered by kv group:
// [group][map][head within the group] (the order in which grouped-query attention takes the query heads when each map's
// keys are a kv head of their own).  Per head: o = a1 - lambda * a2, o / sqrt(mean(o^2) + eps) * post, times
// sigmoid(gate) if a gate is given; out [t, heads * vdim] in the heads' own order.  A warp per (t, head); float32.
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(T* __restrict__ out, const T* __restrict__ a, long long a_stride, const T* __restrict__ gate,
                    long long gate_stride, long long items, int heads, int per_group, int vdim, float lambda, float post,
                    float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = (int)(item % heads);
  const int first = (h / per_group) * 2 * per_group + h % per_group;
  const T* a1 = a + (size_t)t * a_stride + (size_t)first * vdim;
  const T* a2 = a1 + (size_t)per_group * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) {
    const float o = fmaf(-lambda, to_f32(a2[c]), to_f32(a1[c]));
    ss = fmaf(o, o, ss);
  }
  const float r = post / sqrtf(warp_sum(ss) / (float)vdim + eps);
  const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
  for (int c = lane; c < vdim; c += 32) {
    float y = fmaf(-lambda, to_f32(a2[c]), to_f32(a1[c])) * r;
    if (g) y *= 1.f / (1.f + expf(-to_f32(g[c])));
    out[(size_t)item * vdim + c] = from_f32<T>(y);
  }
}

LLMK_API int llmk_diff_combine(void* out, const void* a, long long a_stride, const void* gate, long long gate_stride,
                               int n_tokens, int heads, int per_group, int vdim, float lambda, float post, float eps,
                               int dtype, cudaStream_t stream) {
  const long long items = (long long)n_tokens * heads;
  if (items == 0) return 0;
  LLMK_REQUIRE(per_group > 0 && heads % per_group == 0 && vdim > 0, "diff_combine: %d heads in groups of %d", heads, per_group);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(diff_combine_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (T*)out, (const T*)a,
                  a_stride, (const T*)gate, gate_stride, items, heads, per_group, vdim, lambda, post, eps);
    LLMK_LAUNCH_CHECK("diff_combine");
  });
}

// ---- a scaled sum of two rows ---------------------------------------------------------
// out = sa * a + sb * b row by row (two mixers side by side); a and b tensors or split-K partial results.
template <typename T>
__global__ void __launch_bounds__(256)
scaled_sum_kernel(T* __restrict__ out, MaybePartial<T> a, MaybePartial<T> b, float sa, float sb, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(fmaf(sa, a.at(i), sb * b.at(i)));
}

LLMK_API int llmk_scaled_sum(void* out, const void* a, const float* a_parts, int a_splits, long long a_stride, const void* b,
                             const float* b_parts, int b_splits, long long b_stride, float sa, float sb, int rows, int width,
                             int dtype, cudaStream_t stream) {
  const size_t total = (size_t)rows * width;
  if (total == 0) return 0;
  LLMK_REQUIRE((a != nullptr) != (a_parts != nullptr) && (b != nullptr) != (b_parts != nullptr), "scaled_sum: give each side as a tensor or as partials");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> ma{(const T*)a, a_parts, a_splits, a_stride}, mb{(const T*)b, b_parts, b_splits, b_stride};
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)llmk_sm_count() * 32) blocks = (size_t)llmk_sm_count() * 32;
    launch_kernel(scaled_sum_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, ma, mb, sa, sb, total);
    LLMK_LAUNCH_CHECK("scaled_sum");
  });
}

// ---- clamped gated unit ---------------------------------------------------------------
// out = g * sigmoid(alpha g) * (u + 1) with g = min(gate + b_g, limit), u = clamp(up + b_u, -limit, limit); in holds
// [gate | up] per row (a tensor or split-K partial results), bias float32 [2 * inter] or null.  float32 arithmetic.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, MaybePartial<T> in, const float* __restrict__ bias, int inter,
                                   float limit, float alpha, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i % inter;
    float g = in.at(r * 2 * inter + c), u = in.at(r * 2 * inter + inter + c);
    if (bias) { g += bias[c]; u += bias[inter + c]; }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[i] = from_f32<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

// The same, eight consecutive columns a thread with 16-byte accesses (inter a multiple of 8, aligned bases).
template <typename T>
__global__ void __launch_bounds__(256)
clamped_glu_vec_kernel(T* __restrict__ out, MaybePartial<T> in, const float* __restrict__ bias, int inter, float limit,
                       float alpha, size_t groups) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = inter / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per_row, c = (i % per_row) * 8;
    float g[8], u[8], y[8];
    in.at8(r * 2 * inter + c, g);
    in.at8(r * 2 * inter + inter + c, u);
    if (bias) {
      float bg[8], bu[8];
      Vec8<float>::load(bias + c, bg);
      Vec8<float>::load(bias + inter + c, bu);
#pragma unroll
      for (int k = 0; k < 8; ++k) { g[k] += bg[k]; u[k] += bu[k]; }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gg = fminf(g[k], limit), uu = fminf(fmaxf(u[k], -limit), limit);
      y[k] = gg / (1.f + expf(-alpha * gg)) * (uu + 1.f);
    }
    Vec8<T>::store(out + r * inter + c, y);
  }
}

LLMK_API int llmk_clamped_glu(void* out, const void* gate_up, const float* partials, int splits, long long split_stride,
                              const float* bias, int rows, int inter, float limit, float alpha, int dtype, cudaStream_t stream) {
  const long long total = (long long)rows * inter;
  if (total == 0) return 0;
  LLMK_REQUIRE((gate_up != nullptr) != (partials != nullptr), "clamped_glu: give gate_up or partials");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> x{(const T*)gate_up, partials, splits, split_stride};
    if (inter % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)partials % 16 == 0 &&
        split_stride % 4 == 0 && (uintptr_t)bias % 16 == 0) {
      long long vblocks = (total / 8 + 255) / 256;
      if (vblocks > 65535 * 16) vblocks = 65535 * 16;
      launch_kernel(clamped_glu_vec_kernel<T>, dim3((unsigned)vblocks), dim3(256), 0, stream, (T*)out, x, bias, inter, limit, alpha,
                    (size_t)(total / 8));
      LLMK_LAUNCH_CHECK("clamped_glu");
    }
    long long blocks = (total + 255) / 256;
    if (blocks > 65535 * 16) blocks = 65535 * 16;
    launch_kernel(clamped_glu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, x, bias, inter, limit, alpha,
                  (size_t)total);
    LLMK_LAUNCH_CHECK("clamped_glu");
  });
}
