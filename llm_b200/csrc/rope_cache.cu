// Rotate-half RoPE on q and k, and the write of k and v into the paged cache.
//
// The reference does this in the epilogue of its QKV product
// (kernel/Gemm/QKVGemm.h:27-63): (a, b) = (x_i, x_{i+HS/2}),
// y_i = a*cos - b*sin, y_{i+HS/2} = a*sin + b*cos with float32 tables
// (kernel/embedding/RoPECache.h:15-20), k and v stored at the physical place that
// the step's metadata names (runtime/Engine.h:62-67).  This stand-alone form serves
// every size; the cache layout is [page][kv_head][token in page][head_dim].
#include "common.cuh"

namespace {

template <typename T, bool VEC>
__global__ void rope_kv_write_kernel(MaybePartial<T> src, long long src_stride, T* __restrict__ q_out,
                                     long long q_out_stride,
                                     const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                     int rot_half, const int* __restrict__ positions,
                                     const int* __restrict__ slot_map, T* __restrict__ k_pages,
                                     T* __restrict__ v_pages, int n_heads, int n_kv, int head_dim,
                                     int page_size) {
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_map[t];
  const int page = slot / page_size, off = slot % page_size;
  const size_t row = (size_t)t * src_stride;
  T* q_row = q_out + (size_t)t * q_out_stride;
  const int half = head_dim / 2;
  const float* cs = cos_table ? cos_table + (size_t)pos * rot_half : nullptr;
  const float* sn = cos_table ? sin_table + (size_t)pos * rot_half : nullptr;
  if (VEC) {
    // eight pairs per thread: half is a multiple of 8 because head_dim is a multiple of 16
    const int per_head = half / 8;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    for (int idx = tid; idx < (n_heads + n_kv) * per_head; idx += stride) {
      const int head = idx / per_head, i = (idx % per_head) * 8;
      const size_t h = row + (size_t)head * head_dim;
      float a[8], b[8], c[8], s[8], ya[8], yb[8];
      src.at8(h + i, a);
      src.at8(h + i + half, b);
      if (cs) {
        Vec8<float>::load(cs + i, c);
        Vec8<float>::load(sn + i, s);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) { c[k] = 1.f; s[k] = 0.f; }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) { ya[k] = a[k] * c[k] - b[k] * s[k]; yb[k] = a[k] * s[k] + b[k] * c[k]; }
      T* dst = head < n_heads ? q_row + (size_t)head * head_dim
                              : k_pages + (((size_t)page * n_kv + (head - n_heads)) * page_size + off) * head_dim;
      Vec8<T>::store(dst + i, ya);
      Vec8<T>::store(dst + i + half, yb);
    }
    const size_t v = row + (size_t)(n_heads + n_kv) * head_dim;
    for (int idx = tid * 8; idx < n_kv * head_dim; idx += stride * 8) {
      const int g = idx / head_dim, d = idx % head_dim;
      float x[8];
      src.at8(v + idx, x);
      Vec8<T>::store(v_pages + (((size_t)page * n_kv + g) * page_size + off) * head_dim + d, x);
    }
    return;
  }
  const int rot_items = (n_heads + n_kv) * half;
  for (int idx = threadIdx.x; idx < rot_items; idx += blockDim.x) {
    const int head = idx / half, i = idx % half;
    const size_t h = row + (size_t)head * head_dim;
    const float a = src.at(h + i), b = src.at(h + i + half);
    const float c = cs ? cs[i] : 1.f, s = cs ? sn[i] : 0.f;
    const T ya = from_f32<T>(a * c - b * s), yb = from_f32<T>(a * s + b * c);
    if (head < n_heads) {
      q_row[(size_t)head * head_dim + i] = ya;
      q_row[(size_t)head * head_dim + i + half] = yb;
    } else {
      const int g = head - n_heads;
      T* dst = k_pages + (((size_t)page * n_kv + g) * page_size + off) * head_dim;
      dst[i] = ya;
      dst[i + half] = yb;
    }
  }
  const size_t v = row + (size_t)(n_heads + n_kv) * head_dim;
  for (int idx = threadIdx.x; idx < n_kv * head_dim; idx += blockDim.x) {
    const int g = idx / head_dim, d = idx % head_dim;
    v_pages[(((size_t)page * n_kv + g) * page_size + off) * head_dim + d] = from_f32<T>(src.at(v + idx));
  }
}

}  // namespace

// A row of the source holds q heads, then k heads, then v heads; the source is qkv
// [n_tokens, src_stride] of the element kind, or the float32 partial results
// [splits][n_tokens][src_stride] of a split-K product.  Rotated q goes to q_out (which may be
// the source itself: every pair is read and written by one thread), rotated k and plain v go
// to the pages.  Tables are [max_position, head_dim/2]; without tables (null) nothing is
// rotated and k, v are only stored.
LLMK_API int llmk_rope_kv_write(const void* qkv, const float* partials, int splits, long long split_stride,
                                long long src_stride, void* q_out, long long q_out_stride, const float* cos_table,
                                const float* sin_table, const int* positions, const int* slot_map,
                                void* k_pages, void* v_pages, int n_tokens, int n_heads, int n_kv,
                                int head_dim, int page_size, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(head_dim % 2 == 0, "rope_kv_write: head_dim %d must be even", head_dim);
  LLMK_REQUIRE((qkv != nullptr) != (partials != nullptr), "rope_kv_write: give qkv or partials");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> src{(const T*)qkv, partials, splits, split_stride};
    const bool vec = head_dim % 16 == 0 && src.vector_ok() && src_stride % 8 == 0 && q_out_stride % 8 == 0 &&
                     (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 &&
                     (uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0;
    auto kern = vec ? rope_kv_write_kernel<T, true> : rope_kv_write_kernel<T, false>;
    // few tokens: spread a token's heads over several CTAs (the vector path strides over blockIdx.y)
    const int items = (n_heads + n_kv) * (head_dim / 16);
    const int ys = (vec && n_tokens < 64) ? (items + 63) / 64 : 1;
    launch_kernel(kern, dim3(n_tokens, ys), dim3(vec && ys > 1 ? 64 : 128), 0, stream, src, src_stride, (T*)q_out,
                  q_out_stride, cos_table, sin_table, head_dim / 2, positions, slot_map, (T*)k_pages, (T*)v_pages,
                  n_heads, n_kv, head_dim, page_size);
    LLMK_LAUNCH_CHECK("rope_kv_write");
  });
}

// ---- rotation of neighbouring pairs, from frequencies -------------------------------------
// The other common layout of RoPE: channels 2i and 2i+1 of a head form a pair (not i and i + HS/2),
// only the first 2 * rot_pairs channels of a head turn, and the angle is position * freqs[i], one
// float32 product, with freqs given by the caller (so any scaling of the frequencies is the caller's
// business and no table bounds the position).  Keys and values may differ in size: a row of the
// source holds n_heads * dim query channels, n_kv * dim key channels, n_kv * vdim value channels.
namespace {

template <typename T>
__global__ void __launch_bounds__(128)
rope_pairs_kv_write_kernel(MaybePartial<T> src, long long src_stride, T* __restrict__ q_out, long long q_out_stride,
                           const float* __restrict__ freqs, int rot_pairs, const int* __restrict__ positions,
                           const int* __restrict__ slot_map, T* __restrict__ k_pages, T* __restrict__ v_pages,
                           int n_heads, int n_kv, int dim, int vdim, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const size_t row = (size_t)t * src_stride;
  T* q_row = q_out + (size_t)t * q_out_stride;
  size_t k_base = 0, v_base = 0;
  if (n_kv) {
    const int slot = slot_map[t];
    const size_t page = slot / page_size, off = slot % page_size;
    k_base = (page * n_kv * page_size + off) * dim;           // + g * page_size * dim
    v_base = (page * n_kv * page_size + off) * vdim;
  }
  const int pairs = (dim + 1) / 2;
  for (int idx = threadIdx.x; idx < (n_heads + n_kv) * pairs; idx += blockDim.x) {
    const int head = idx / pairs, i = idx % pairs;
    const int d0 = 2 * i, d1 = d0 + 1;
    const size_t h = row + (size_t)head * dim;
    float a = src.at(h + d0), b = d1 < dim ? src.at(h + d1) : 0.f;
    if (i < rot_pairs && d1 < dim) {
      float s, c;
      sincosf(pos * freqs[i], &s, &c);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    T* dst = head < n_heads ? q_row + (size_t)head * dim
                            : k_pages + k_base + (size_t)(head - n_heads) * page_size * dim;
    dst[d0] = from_f32<T>(a);
    if (d1 < dim) dst[d1] = from_f32<T>(b);
  }
  const size_t v = row + (size_t)(n_heads + n_kv) * dim;
  for (int idx = threadIdx.x; idx < n_kv * vdim; idx += blockDim.x) {
    const int g = idx / vdim, d = idx % vdim;
    v_pages[v_base + (size_t)g * page_size * vdim + d] = from_f32<T>(src.at(v + idx));
  }
}


// ---- norm over the whole projection, rotation by computed angles, store ----------------------------------------
// One CTA per token: sums the split-K partial results, takes the RMS norm of the token's whole q projection
// (n_heads * dim numbers at once, weights q_gain) and of its whole k projection (n_kv * dim, weights k_gain) before they
// are split into heads (either gain null: that side is not normed), turns the first 2 * rot_pairs channels of every q and k
// head by position * freqs[i], channel i against channel i + rot_pairs (halves) or 2i against 2i + 1 (neighbours), and
// stores k and v at the token's slot.  The row is held in shared memory as float32.
template <typename T>
__global__ void __launch_bounds__(256)
norm_rope_kv_write_kernel(MaybePartial<T> src, long long src_stride, T* __restrict__ q_out, long long q_out_stride,
                          const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                          const float* __restrict__ freqs, int rot_pairs, int halves, const int* __restrict__ positions,
                          const int* __restrict__ slot_map, T* __restrict__ k_pages, T* __restrict__ v_pages,
                          int n_heads, int n_kv, int dim, int vdim, int page_size) {
  extern __shared__ float row_s[];            // [(n_heads + n_kv) * dim]
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const size_t row = (size_t)t * src_stride;
  const int qn = n_heads * dim, kn = n_kv * dim;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < qn + kn; c += blockDim.x) {
    const float v = src.at(row + c);
    row_s[c] = v;
    if (c < qn) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
  }
  const float tq = block_sum(sq, red);
  const float tk = block_sum(sk, red);
  const float rq = q_gain ? 1.f / sqrtf(tq / (float)qn + eps) : 1.f;
  const float rk = (k_gain && kn) ? 1.f / sqrtf(tk / (float)kn + eps) : 1.f;
  size_t k_base = 0, v_base = 0;
  if (n_kv) {
    const int slot = slot_map[t];
    const size_t page = slot / page_size, off = slot % page_size;
    k_base = (page * n_kv * page_size + off) * dim;
    v_base = (page * n_kv * page_size + off) * vdim;
  }
  T* q_row = q_out + (size_t)t * q_out_stride;
  // every channel belongs to one item: a turning pair (two channels) or a channel that passes
  const int per_head = dim - rot_pairs;       // rot_pairs pairs + (dim - 2 rot_pairs) single channels
  for (int idx = threadIdx.x; idx < (n_heads + n_kv) * per_head; idx += blockDim.x) {
    const int head = idx / per_head, i = idx % per_head;
    const bool is_q = head < n_heads;
    const float r = is_q ? rq : rk;
    const float* gain = is_q ? q_gain : k_gain;
    const int c_base = head * dim;             // column of the head in the row (q heads first, then k heads)
    const int g_base = is_q ? c_base : c_base - qn;
    T* dst = is_q ? q_row + (size_t)head * dim : k_pages + k_base + (size_t)(head - n_heads) * page_size * dim;
    if (i < rot_pairs) {
      const int d0 = halves ? i : 2 * i, d1 = halves ? i + rot_pairs : 2 * i + 1;
      const float a = row_s[c_base + d0] * r * (gain ? gain[g_base + d0] : 1.f);
      const float b = row_s[c_base + d1] * r * (gain ? gain[g_base + d1] : 1.f);
      float sn, cs;
      sincosf(pos * freqs[i], &sn, &cs);
      dst[d0] = from_f32<T>(a * cs - b * sn);
      dst[d1] = from_f32<T>(b * cs + a * sn);
    } else {
      const int d = i + rot_pairs;
      dst[d] = from_f32<T>(row_s[c_base + d] * r * (gain ? gain[g_base + d] : 1.f));
    }
  }
  const size_t v = row + (size_t)(qn + kn);
  for (int idx = threadIdx.x; idx < n_kv * vdim; idx += blockDim.x) {
    const int g = idx / vdim, d = idx % vdim;
    v_pages[v_base + (size_t)g * page_size * vdim + d] = from_f32<T>(src.at(v + idx));
  }
}

// ---- norm per head with one shared weight, store; k and v with head counts of their own ----------------------
// A row holds n_q query heads and n_k key heads of dim numbers, then n_v value heads of vdim.  Every q and k head is
// divided by its own root mean square (eps inside the root) and multiplied by gain [dim], one weight vector for all of them
// (null: the heads pass as they are); q goes to q_out, k and v to the token's slot in their pages, which may hold different
// numbers of heads (several attention maps over one set of values).  A warp per head; sums in float32.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kv_write_kernel(MaybePartial<T> src, long long src_stride, T* __restrict__ q_out, long long q_out_stride,
                          const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                          const int* __restrict__ slot_map, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q, int n_k,
                          int n_v, int dim, int vdim, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const size_t row = (size_t)t * src_stride;
  size_t page = 0, off = 0;
  if (n_k || n_v) {
    const int slot = slot_map[t];
    page = slot / page_size; off = slot % page_size;
  }
  for (int head = warp; head < n_q + n_k; head += warps) {
    const bool is_q = head < n_q;
    const float* gain = is_q ? q_gain : k_gain;
    const size_t c0 = row + (size_t)head * dim;
    float ss = 0.f;
    if (gain)
      for (int d = lane; d < dim; d += 32) { const float v = src.at(c0 + d); ss = fmaf(v, v, ss); }
    const float r = gain ? 1.f / sqrtf(warp_sum(ss) / (float)dim + eps) : 1.f;
    T* dst = is_q ? q_out + (size_t)t * q_out_stride + (size_t)head * dim
                  : k_pages + ((page * n_k + (head - n_q)) * page_size + off) * dim;
    for (int d = lane; d < dim; d += 32) dst[d] = from_f32<T>(gain ? src.at(c0 + d) * r * gain[d] : src.at(c0 + d));
  }
  const size_t v0 = row + (size_t)(n_q + n_k) * dim;
  for (int idx = threadIdx.x; idx < n_v * vdim; idx += blockDim.x) {
    const int g = idx / vdim, d = idx % vdim;
    v_pages[((page * n_v + g) * page_size + off) * vdim + d] = from_f32<T>(src.at(v0 + idx));
  }
}

}  // namespace

// qkv / partials as in llmk_rope_kv_write; q_out may be the source itself (a pair is read and written by
// one thread).  freqs float32 [rot_pairs]; k_pages [pages, n_kv, page_size, dim], v_pages [.., vdim];
// n_kv 0: only the queries are rotated and nothing is stored.
LLMK_API int llmk_rope_pairs_kv_write(const void* qkv, const float* partials, int splits, long long split_stride,
                                      long long src_stride, void* q_out, long long q_out_stride, const float* freqs,
                                      int rot_pairs, const int* positions, const int* slot_map, void* k_pages,
                                      void* v_pages, int n_tokens, int n_heads, int n_kv, int dim, int vdim,
                                      int page_size, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE((qkv != nullptr) != (partials != nullptr), "rope_pairs_kv_write: give qkv or partials");
  LLMK_REQUIRE(rot_pairs >= 0 && 2 * rot_pairs <= dim, "rope_pairs_kv_write: %d pairs do not fit a head of %d", rot_pairs, dim);
  LLMK_REQUIRE(rot_pairs == 0 || freqs != nullptr, "rope_pairs_kv_write: frequencies are missing");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> src{(const T*)qkv, partials, splits, split_stride};
    launch_kernel(rope_pairs_kv_write_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, src, src_stride, (T*)q_out,
                  q_out_stride, freqs, rot_pairs, positions, slot_map, (T*)k_pages, (T*)v_pages, n_heads, n_kv, dim,
                  vdim, page_size);
    LLMK_LAUNCH_CHECK("rope_pairs_kv_write");
  });
}

// As llmk_rope_pairs_kv_write, with the RMS norm of the whole q and k projections first (gains float32 [n_heads * dim] and
// [n_kv * dim], each may be null) and the choice of the pairs: halves != 0 turns channel i against i + rot_pairs.
LLMK_API int llmk_norm_rope_kv_write(const void* qkv, const float* partials, int splits, long long split_stride,
                                     long long src_stride, void* q_out, long long q_out_stride, const float* q_gain,
                                     const float* k_gain, float eps, const float* freqs, int rot_pairs, int halves,
                                     const int* positions, const int* slot_map, void* k_pages, void* v_pages, int n_tokens,
                                     int n_heads, int n_kv, int dim, int vdim, int page_size, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE((qkv != nullptr) != (partials != nullptr), "norm_rope_kv_write: give qkv or partials");
  LLMK_REQUIRE(rot_pairs >= 0 && 2 * rot_pairs <= dim, "norm_rope_kv_write: %d pairs do not fit a head of %d", rot_pairs, dim);
  LLMK_REQUIRE(rot_pairs == 0 || freqs != nullptr, "norm_rope_kv_write: frequencies are missing");
  const size_t smem = (size_t)(n_heads + n_kv) * dim * sizeof(float);
  LLMK_REQUIRE(smem <= 200 * 1024, "norm_rope_kv_write: a projection of %d numbers does not fit shared memory", (n_heads + n_kv) * dim);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> src{(const T*)qkv, partials, splits, split_stride};
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_rope_kv_write_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(norm_rope_kv_write_kernel<T>, dim3(n_tokens), dim3(256), smem, stream, src, src_stride, (T*)q_out,
                  q_out_stride, q_gain, k_gain, eps, freqs, rot_pairs, halves, positions, slot_map, (T*)k_pages, (T*)v_pages,
                  n_heads, n_kv, dim, vdim, page_size);
    LLMK_LAUNCH_CHECK("norm_rope_kv_write");
  });
}

// qkv / partials as in llmk_rope_kv_write: a row of n_q * dim | n_k * dim | n_v * vdim numbers.  q_gain, k_gain float32
// [dim] (null: no norm on that side); k_pages [pages, n_k, page_size, dim], v_pages [pages, n_v, page_size, vdim].
LLMK_API int llmk_head_norm_kv_write(const void* qkv, const float* partials, int splits, long long split_stride,
                                     long long src_stride, void* q_out, long long q_out_stride, const float* q_gain,
                                     const float* k_gain, float eps, const int* slot_map, void* k_pages, void* v_pages,
                                     int n_tokens, int n_q, int n_k, int n_v, int dim, int vdim, int page_size, int dtype,
                                     cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE((qkv != nullptr) != (partials != nullptr), "head_norm_kv_write: give qkv or partials");
  LLMK_REQUIRE(n_q >= 0 && n_k >= 0 && n_v >= 0 && dim > 0 && vdim > 0 && page_size > 0, "head_norm_kv_write: bad sizes");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> src{(const T*)qkv, partials, splits, split_stride};
    launch_kernel(head_norm_kv_write_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, src, src_stride, (T*)q_out, q_out_stride,
                  q_gain, k_gain, eps, slot_map, (T*)k_pages, (T*)v_pages, n_q, n_k, n_v, dim, vdim, page_size);
    LLMK_LAUNCH_CHECK("head_norm_kv_write");
  });
}
