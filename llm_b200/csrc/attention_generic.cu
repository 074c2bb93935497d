// Causal grouped-query attention over the paged cache, any sizes, float32 arithmetic.
//
// One warp owns one (token, query head).  Keys are visited in tiles of 32 that start
// at absolute positions 0, 32, 64, ...: lane j scores key tile+j, the warp keeps a
// running maximum and sum (online softmax), then all lanes add p_j * v_j in key order.
// The order of every sum is a function of the token's own position alone, so a
// token's output does not depend on how the prompt was cut or what shares the batch.
// Visible keys: max(0, pos-window+1) <= j <= pos (window 0 = all), as in the reference
// (kernel/attention/attention_NH_32_NKV_4_HS_64.h:169-172,228-232); scores are scaled
// by the given factor instead of the reference's constant for head size 64 (:197).
// This is the attention of the 32-bit path and of bfloat16 shapes that the tensor-core
// kernels refuse.  Options, all off at zero: values of another size than the keys (vdim); a soft cap
// on the scaled scores, s <- cap * tanh(s / cap); a sink, a key with score 0 and no value that only
// adds 1 to the softmax's denominator; and, with a window, the first keep_first keys of the request,
// which stay visible (at their true positions) after the window has passed them.  Further: the sink's score may be a
// learned number per head (sink_values; it is not scaled); the mask may be by chunks instead of a window (chunk > 0: a
// query sees the keys at or before it whose position has the same floor(position / chunk)); and the weights may be
// sigmoid(score + bias[head]) without a softmax (sigmoid_bias given: no maximum, no normalisation, no sink).
// Two more: a bias that grows with the distance, r1[head] * ln(1 + r2[head] * (position - key position)), taken off the capped
// score; and key heads that share value heads (v_share neighbouring key heads read one value head: several attention maps,
// each with keys of its own, over one set of values).
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HEAD_DIM = 1024;     // the kernel is built for head sizes up to 256, up to 512 and up to 1024

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int head_dim);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k,
                                                int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; d += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(k + d);
    s = fmaf(q[d], kv.x, s);
    s = fmaf(q[d + 1], kv.y, s);
    s = fmaf(q[d + 2], kv.z, s);
    s = fmaf(q[d + 3], kv.w, s);
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; d += 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(k + d);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s = fmaf(q[d + 2 * i], __low2float(p[i]), s);
      s = fmaf(q[d + 2 * i + 1], __high2float(p[i]), s);
    }
  }
  return s;
}

// a row that does not start on a 16-byte boundary, or is no whole number of 16-byte pieces
// (head sizes off the 8-grid in bfloat16, off the 4-grid in float32): element by element
template <typename T>
__device__ __forceinline__ float dot_row_scalar(const float* __restrict__ q, const T* __restrict__ k, int head_dim) {
  float s = 0.f;
  for (int d = 0; d < head_dim; ++d) s = fmaf(q[d], to_f32(k[d]), s);
  return s;
}

template <typename T, int MAXD>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ q,
                               long long q_stride, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int table_width, const int* __restrict__ token_entry,
                               const int* __restrict__ positions, int n_tokens, int n_heads, int n_kv,
                               int head_dim, int vdim, int page_size, int window, int keep_first, float scale,
                               float softcap, int sink, bool vec, const float* __restrict__ sink_values, int chunk,
                               const float* __restrict__ sigmoid_bias, const float* __restrict__ dist_r1,
                               const float* __restrict__ dist_r2, int v_share) {
  __shared__ float q_s[WARPS][MAXD];
  pdl_launch_dependents();      // let the next kernel start its own prologue now
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), h = (int)(item % n_heads);
  const int g = h / (n_heads / n_kv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_entry[t] * table_width;
  const int lo = chunk > 0 ? (pos / chunk) * chunk : (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int keep_end = min(keep_first, lo);      // keys [0, keep_end) lie before the window and are seen all the same
  const int lo_tile = (lo / 32) * 32;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const float r1 = dist_r1 ? dist_r1[h] : 0.f, r2 = dist_r1 ? dist_r2[h] : 0.f;
  const int n_v = n_kv / v_share, gv = g / v_share;      // v_share neighbouring key heads read one value head

  const T* q_row = q + (size_t)t * q_stride + (size_t)h * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = to_f32(q_row[d]);
  __syncwarp();

  float acc[MAXD / 32];
#pragma unroll
  for (int i = 0; i < MAXD / 32; ++i) acc[i] = 0.f;
  // the sink is the first term of the softmax: score 0, weight exp(0 - m), no value
  const bool gated = sigmoid_bias != nullptr;
  const float bias = gated ? sigmoid_bias[h] : 0.f;
  float m = sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;

  for (int tile = keep_end > 0 ? 0 : lo_tile; tile <= pos; tile += 32) {
    if (tile >= keep_end && tile < lo_tile) {      // between the kept keys and the window: nothing to see
      tile = lo_tile - 32;
      continue;
    }
    const int kp = tile + lane;
    const bool valid = kp <= pos && (kp >= lo || kp < keep_end);
    long long row = 0;                             // the value's place in units of rows of vdim
    float s = -INFINITY;
    if (valid) {
      const int page = table[kp / page_size];
      row = ((long long)page * n_v + gv) * page_size + kp % page_size;
      const T* k_row = k_pages + (((long long)page * n_kv + g) * page_size + kp % page_size) * head_dim;
      s = (vec ? dot_row<T>(q_s[warp], k_row, head_dim) : dot_row_scalar<T>(q_s[warp], k_row, head_dim)) * scale;
      if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
      if (dist_r1) s -= r1 * log1pf(r2 * (float)(pos - kp));      // a bias that grows with the distance to the key
    }
    float p;
    if (gated) {
      p = valid ? 1.f / (1.f + expf(-(s + bias))) : 0.f;
    } else {
      const float m_new = fmaxf(m, warp_max(s));
      const float alpha = expf(m - m_new);  // m = -inf at the first tile gives 0
      p = valid ? expf(s - m_new) : 0.f;
      l = l * alpha + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < MAXD / 32; ++i) acc[i] *= alpha;
    }
    const int n_valid = min(32, pos - tile + 1);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long rj = __shfl_sync(0xffffffffu, row, j);
      if (pj != 0.f) {
        const T* v = v_pages + rj * vdim;
#pragma unroll
        for (int i = 0; i < MAXD / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < vdim) acc[i] = fmaf(pj, to_f32(v[d]), acc[i]);
        }
      }
    }
  }
  const float inv = gated ? 1.f : 1.f / l;
  T* o = out + (size_t)t * out_stride + (size_t)h * vdim;
#pragma unroll
  for (int i = 0; i < MAXD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) o[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

// q [n_tokens, q_stride] with head h at column h*head_dim; out [n_tokens, out_stride] with head h at column
// h*vdim.  k_pages [pages, n_kv, page_size, head_dim], v_pages [pages, n_kv, page_size, vdim]; block_table [entries, table_width] holds,
// for batch entry e, the page of positions [i*page_size, (i+1)*page_size) at column i.
// Further options: dist_r1, dist_r2 (float32 [heads], both or neither): r1[h] * ln(1 + r2[h] * (query position - key
// position)) is taken off every score after the cap; v_share > 1: v_pages has n_kv / v_share heads and the key heads
// v_share * i .. v_share * i + v_share - 1 read value head i (several attention maps over one set of values).
LLMK_API int llmk_paged_attention_generic_ex(void* out, long long out_stride, const void* q, long long q_stride,
                                             const void* k_pages, const void* v_pages, const int* block_table,
                                             int table_width, const int* token_entry, const int* positions,
                                             int n_tokens, int n_heads, int n_kv, int head_dim, int vdim, int page_size,
                                             int window, int keep_first, float scale, float softcap, int sink, int dtype,
                                             cudaStream_t stream, const float* sink_values, int chunk, const float* sigmoid_bias,
                                             const float* dist_r1, const float* dist_r2, int v_share) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(v_share >= 1 && n_kv % v_share == 0, "paged_attention: %d key heads do not share values in runs of %d", n_kv, v_share);
  LLMK_REQUIRE((dist_r1 != nullptr) == (dist_r2 != nullptr), "paged_attention: the distance bias takes both of its numbers");
  LLMK_REQUIRE(head_dim > 0 && head_dim <= MAX_HEAD_DIM, "paged_attention: head_dim %d must be 1 to %d", head_dim, MAX_HEAD_DIM);
  LLMK_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "paged_attention: %d query heads do not divide into %d kv heads",
               n_heads, n_kv);
  LLMK_REQUIRE(vdim > 0 && vdim <= MAX_HEAD_DIM, "paged_attention: value size %d must be 1 to %d", vdim, MAX_HEAD_DIM);
  LLMK_REQUIRE(page_size > 0 && window >= 0, "paged_attention: bad page_size %d or window %d", page_size, window);
  LLMK_REQUIRE(keep_first >= 0 && softcap >= 0.f, "paged_attention: bad keep_first %d or soft cap %f", keep_first, (double)softcap);
  LLMK_REQUIRE(chunk >= 0 && !(chunk > 0 && keep_first > 0), "paged_attention: bad chunk %d", chunk);
  if (sigmoid_bias) sink = 0;
  if (window == 0) keep_first = 0;
  const int widest = head_dim > vdim ? head_dim : vdim;
  const long long items = (long long)n_tokens * n_heads;
  const long long blocks = (items + WARPS - 1) / WARPS;
  LLMK_REQUIRE(blocks < (1ll << 31), "paged_attention: too many (token, head) items");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    const bool vec = head_dim % (16 / (int)sizeof(T)) == 0 && (uintptr_t)k_pages % 16 == 0;      // whole 16-byte pieces per key row
    if (widest <= 256)
      launch_kernel(paged_attention_generic_kernel<T, 256>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
          (T*)out, out_stride, (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table,
          table_width, token_entry, positions, n_tokens, n_heads, n_kv, head_dim, vdim, page_size, window, keep_first, scale,
          softcap, sink, vec, sink_values, chunk, sigmoid_bias, dist_r1, dist_r2, v_share);
    else if (widest <= 512)      // the wide head of a latent attention (its rank)
      launch_kernel(paged_attention_generic_kernel<T, 512>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
          (T*)out, out_stride, (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table,
          table_width, token_entry, positions, n_tokens, n_heads, n_kv, head_dim, vdim, page_size, window, keep_first, scale,
          softcap, sink, vec, sink_values, chunk, sigmoid_bias, dist_r1, dist_r2, v_share);
    else
      launch_kernel(paged_attention_generic_kernel<T, MAX_HEAD_DIM>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
          (T*)out, out_stride, (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table,
          table_width, token_entry, positions, n_tokens, n_heads, n_kv, head_dim, vdim, page_size, window, keep_first, scale,
          softcap, sink, vec, sink_values, chunk, sigmoid_bias, dist_r1, dist_r2, v_share);
    LLMK_LAUNCH_CHECK("paged_attention_generic");
  });
}

LLMK_API int llmk_paged_attention_generic(void* out, long long out_stride, const void* q, long long q_stride,
                                          const void* k_pages, const void* v_pages, const int* block_table,
                                          int table_width, const int* token_entry, const int* positions,
                                          int n_tokens, int n_heads, int n_kv, int head_dim, int vdim, int page_size,
                                          int window, int keep_first, float scale, float softcap, int sink, int dtype,
                                          cudaStream_t stream, const float* sink_values, int chunk, const float* sigmoid_bias) {
  return llmk_paged_attention_generic_ex(out, out_stride, q, q_stride, k_pages, v_pages, block_table, table_width, token_entry,
                                         positions, n_tokens, n_heads, n_kv, head_dim, vdim, page_size, window, keep_first, scale,
                                         softcap, sink, dtype, stream, sink_values, chunk, sigmoid_bias, nullptr, nullptr, 1);
}
