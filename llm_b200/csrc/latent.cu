// The cached side of a latent attention: a token's compressed key/value vector.
//
// A layer with a down-projection of its own turns each token's projection (rank numbers) into
// c = x / sqrt(mean(x^2) + eps) * gain and keeps only c, in a paged cache with one "head" of
// size rank and no separate values.  Keys and values of every head are linear maps of c, so the
// attention itself runs on c: the queries are first carried through the key map
// (q'_h = Wuk_h^T q_h, so that q_h . k_h = q'_h . c), the attention is then a multi-query one whose
// keys and values are both c, and its result is carried through the value map afterwards.  This
// file holds the norm-and-store step; the two per-head maps are batched products (gemm_simt.cu)
// and the attention is the paged multi-query kernels that the other mixers use.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

// One warp per token: sum of squares, reciprocal root and scaling in float32; the result is
// rounded to the cache's element type once and written at the token's place in the pages.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_norm_store_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ gain, float eps,
                         const int* __restrict__ slot_map, T* __restrict__ pages, int n_tokens, int rank, int row_width) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= n_tokens) return;
  const T* row = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float v = to_f32(row[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)rank + eps);
  T* dst = pages + (size_t)slot_map[t] * row_width;
  for (int c = lane; c < rank; c += 32) dst[c] = from_f32<T>(to_f32(row[c]) * r * gain[c]);
  for (int c = rank + lane; c < row_width; c += 32) dst[c] = from_f32<T>(0.f);      // a row wider than the rank ends in zeros
}


// The same for a latent attention with a query latent and a rotated key part: one warp per token takes the token's
// projection x = [query latent: q_rank | key/value latent: rank | rotated key part: rot] (float32) and writes
//   cq = rms(x_q) * q_gain                                        to cq_out (the element kind of the step), and
//   [rotated key part | rms(x_c) * gain | zeros]                   to the token's cache row:
// the pairs (2i, 2i + 1), i < pairs, of the key part turn by position * freqs[i] (one float32 product, sincosf); what lies
// beyond them passes.  The rotated part comes first in the row so that the kernels that turn the leading channels of a
// head serve the queries too.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_rope_norm_store_kernel(const float* __restrict__ x, long long x_stride, const float* __restrict__ q_gain, int q_rank,
                              T* __restrict__ cq_out, long long cq_stride, const float* __restrict__ gain, int rank, int rot,
                              const float* __restrict__ freqs, int pairs, const int* __restrict__ positions, float eps,
                              const int* __restrict__ slot_map, T* __restrict__ pages, int n_tokens, int row_width) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= n_tokens) return;
  const float* row = x + (size_t)t * x_stride;
  if (q_rank > 0) {
    float ss = 0.f;
    for (int c = lane; c < q_rank; c += 32) ss = fmaf(row[c], row[c], ss);
    const float r = 1.f / sqrtf(warp_sum(ss) / (float)q_rank + eps);
    for (int c = lane; c < q_rank; c += 32) cq_out[(size_t)t * cq_stride + c] = from_f32<T>(row[c] * r * q_gain[c]);
  }
  if (pages == nullptr) return;
  const float* lat = row + q_rank;
  const float* kr = lat + rank;
  float ss = 0.f;
  for (int c = lane; c < rank; c += 32) ss = fmaf(lat[c], lat[c], ss);
  const float r = 1.f / sqrtf(warp_sum(ss) / (float)rank + eps);
  T* dst = pages + (size_t)slot_map[t] * row_width;
  const float pos = (float)positions[t];
  for (int i = lane; i < rot / 2; i += 32) {
    float u = kr[2 * i], v = kr[2 * i + 1];
    if (i < pairs) {
      float sn, cs;
      sincosf(pos * freqs[i], &sn, &cs);
      const float u2 = u * cs - v * sn, v2 = v * cs + u * sn;
      u = u2; v = v2;
    }
    dst[2 * i] = from_f32<T>(u);
    dst[2 * i + 1] = from_f32<T>(v);
  }
  for (int c = lane; c < rank; c += 32) dst[rot + c] = from_f32<T>(lat[c] * r * gain[c]);
  for (int c = rot + rank + lane; c < row_width; c += 32) dst[c] = from_f32<T>(0.f);
}

}  // namespace

// x [n_tokens, x_stride]: the first `rank` columns of a row are the token's projection.
// pages [pages, 1, page_size, row_width] with row_width >= rank (a cache whose rows are padded to a width
// that the attention kernels take; the padding is written as zeros); slot_map[t] = page * page_size + offset.
LLMK_API int llmk_latent_norm_store(const void* x, long long x_stride, const float* gain, float eps,
                                    const int* slot_map, void* pages, int n_tokens, int rank, int row_width, int dtype,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(rank > 0 && x_stride >= rank && row_width >= rank, "latent_norm_store: bad rank %d, width %d or stride %lld", rank, row_width, x_stride);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(latent_norm_store_kernel<T>, dim3((n_tokens + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream,
                  (const T*)x, x_stride, gain, eps, slot_map, (T*)pages, n_tokens, rank, row_width);
    LLMK_LAUNCH_CHECK("latent_norm_store");
  });
}

// x float32 [n_tokens, x_stride]: [q_rank | rank | rot] per row (q_rank 0: no query latent; pages null: no cache row, a
// layer that reads another's).  rot is even; pairs <= rot / 2.  pages [pages, 1, page_size, row_width], row_width >= rot + rank.
LLMK_API int llmk_latent_rope_norm_store(const float* x, long long x_stride, const float* q_gain, int q_rank, void* cq_out,
                                         long long cq_stride, const float* gain, int rank, int rot, const float* freqs, int pairs,
                                         const int* positions, float eps, const int* slot_map, void* pages, int n_tokens,
                                         int row_width, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(rank > 0 && rot >= 0 && rot % 2 == 0 && 2 * pairs <= rot && q_rank >= 0,
               "latent_rope_norm_store: bad rank %d, rotated size %d, pairs %d or query rank %d", rank, rot, pairs, q_rank);
  LLMK_REQUIRE(pages == nullptr || row_width >= rot + rank, "latent_rope_norm_store: a row of %d is too narrow", row_width);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(latent_rope_norm_store_kernel<T>, dim3((n_tokens + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream, x, x_stride,
                  q_gain, q_rank, (T*)cq_out, cq_stride, gain, rank, rot, freqs, pairs, positions, eps, slot_map, (T*)pages,
                  n_tokens, row_width);
    LLMK_LAUNCH_CHECK("latent_rope_norm_store");
  });
}
