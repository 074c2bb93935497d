// A routed feed-forward (mixture of experts): router, grouping of the tokens by expert, the
// experts' two products over the groups, and the weighted sum.
//
//   route    z = h Wr^T + b with float32 accumulation (the engine's product kernels make h Wr^T); the
//            `top` largest z of a token (ties to the lower index); their weights are the softmax
//            over those `top` values alone, or (over_all) their shares of the softmax over every
//            expert, which then do not sum to one.
//   group    every (token, choice) pair gets a slot in a list that is sorted by expert, each
//            expert's run padded to whole tiles of 64 slots, so that a tile of the products below
//            belongs to one expert.  The launch sizes depend on the numbers of tokens, choices and
//            experts only: what a step's routing turns out to be is read on the device.
//   products C[slot] = act(A[row of slot] . W[expert of the slot's tile]^T), float32 accumulation in a
//            fixed k order per element, so a pair's result does not depend on its slot or on what
//            else is in the batch.
//   combine  out[t] = shared[t] + sum_j weight[t, j] * y[slot of (t, j)], summed in the order of j.
#include "common.cuh"

namespace {

constexpr int ROUTE_WARPS = 4;
constexpr int MAX_EXPERTS = 256;
constexpr int TILE = 64;          // slots per tile of the grouped products

__device__ __forceinline__ float act_of(float z, int kind) {
  switch (kind) {
    case 0: { const float r = fmaxf(z, 0.f); return r * r; }
    case 1: return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
    case 2: return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    case 3: return z / (1.f + expf(-z));
    default: return z;
  }
}

// One warp per token: its logits (a float32 tensor, or the unsummed partial results of the split-K
// product that made them) plus the bias, then `top` rounds of arg-max over the warp.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
topk_kernel(MaybePartial<float> z, const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
            int n_tokens, int experts, int top, int over_all) {
  __shared__ float z_s[ROUTE_WARPS][MAX_EXPERTS];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  for (int e = lane; e < experts; e += 32) z_s[warp][e] = z.at((size_t)t * experts + e) + (bias ? bias[e] : 0.f);
  __syncwarp();
  float z_max = 0.f, denom = 0.f, denom_all = 0.f;
  if (over_all) {                                     // the softmax's denominator over every expert, before any is struck out
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z_s[warp][e]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < experts; e += 32) s += expf(z_s[warp][e] - mx);
    denom_all = warp_sum(s);
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z_s[warp][e];
      if (v > best) { best = v; arg = e; }            // ascending e: the first of equal values stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > best || (ov == best && oa < arg)) { best = ov; arg = oa; }
    }
    if (j == 0) z_max = best;
    const float p = expf(best - z_max);
    denom += p;
    if (lane == 0) {
      ids[(size_t)t * top + j] = arg < experts ? arg : -1;      // no finite logit left: the pair is dropped
      weights[(size_t)t * top + j] = p;
      if (arg < experts) z_s[warp][arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = 1.f / (over_all ? denom_all : denom);
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] *= inv;
  }
}

// Sigmoid router with groups: scores s = sigmoid(z); the choice is made on s + correction, the weights are the chosen
// experts' s themselves (not renormalised).  The experts form `groups` equal runs of neighbours; a group's score is the sum
// of its two largest choice scores (of its one, in groups of one), and only experts of the `keep` best groups can be chosen:
// the others are struck out (minus infinity, since choice scores may be negative).  Ties go to the lower index, for groups
// and for experts.  One warp per token.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
topk_sigmoid_kernel(MaybePartial<float> z, const float* __restrict__ correction, int* __restrict__ ids,
                    float* __restrict__ weights, int n_tokens, int experts, int top, int groups, int keep) {
  __shared__ float c_s[ROUTE_WARPS][MAX_EXPERTS], s_s[ROUTE_WARPS][MAX_EXPERTS], g_s[ROUTE_WARPS][MAX_EXPERTS];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  for (int e = lane; e < experts; e += 32) {
    const float sc = 1.f / (1.f + expf(-z.at((size_t)t * experts + e)));
    s_s[warp][e] = sc;
    c_s[warp][e] = sc + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (keep < groups) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;               // the largest and the second largest of the group
      for (int i = 0; i < per; ++i) {
        const float v = c_s[warp][g * per + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      g_s[warp][g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // strike out every group but the `keep` best: keep rounds of arg-max mark a group with +infinity
    for (int j = 0; j < keep; ++j) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = g_s[warp][g];
        if (v != INFINITY && v > best) { best = v; arg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ov > best || (ov == best && oa < arg)) { best = ov; arg = oa; }
      }
      if (lane == 0 && arg < groups) g_s[warp][arg] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (g_s[warp][e / per] != INFINITY) c_s[warp][e] = -INFINITY;
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c_s[warp][e];
      if (v > best) { best = v; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ov > best || (ov == best && oa < arg)) { best = ov; arg = oa; }
    }
    if (lane == 0) {
      const bool found = arg < experts;
      ids[(size_t)t * top + j] = found ? arg : -1;              // nothing left to choose: the pair is dropped
      weights[(size_t)t * top + j] = found ? s_s[warp][arg] : 0.f;
      if (found) c_s[warp][arg] = -INFINITY;
    }
    __syncwarp();
  }
}

// One block.  counts -> padded offsets -> slots.  meta[0] = tiles in use.
__global__ void __launch_bounds__(1024)
group_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ meta, int* __restrict__ tile_expert,
             int* __restrict__ slot_src, int* __restrict__ pair_slot, int max_tiles, int TILE) {
  __shared__ int count[MAX_EXPERTS], offset[MAX_EXPERTS], cursor[MAX_EXPERTS];
  __shared__ int total_tiles;
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      offset[e] = tiles * TILE;
      const int n = (count[e] + TILE - 1) / TILE;
      for (int k = 0; k < n && tiles + k < max_tiles; ++k) tile_expert[tiles + k] = e;
      tiles += n;
    }
    total_tiles = tiles < max_tiles ? tiles : max_tiles;
    meta[0] = total_tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < total_tiles * TILE; i += blockDim.x) slot_src[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= experts) { pair_slot[i] = -1; continue; }
    const int slot = offset[e] + atomicAdd(&cursor[e], 1);
    slot_src[slot] = i;
    pair_slot[i] = slot;
  }
}

// x_sorted[slot] = x[token of the slot's pair] (zeros in padding slots): the rows of the tokens in the
// order of the slots, for a grouped product that reads its rows as whole tiles.
template <typename T>
__global__ void gather_rows_by_slot_kernel(T* __restrict__ out, const T* __restrict__ x, long long x_stride,
                                           const int* __restrict__ slot_src, const int* __restrict__ meta, int div,
                                           int cols, int tile) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  if (slot >= meta[0] * tile) return;
  const int src = slot_src[slot];
  T* dst = out + (size_t)slot * cols;
  if (src < 0) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = from_f32<T>(0.f);
    return;
  }
  const T* row = x + (size_t)(src / div) * x_stride;
  constexpr int V = 16 / (int)sizeof(T);
  if (cols % V == 0 && x_stride % V == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(row + c);
    return;
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = row[c];
}

constexpr int BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

// C[slot, :] = act(A[row(slot), :] . W[expert]^T) for the slots of tile blockIdx.y.
// gather_div > 0: row(slot) = slot_src[slot] / gather_div (the token of the pair); 0: row(slot) = slot.
template <typename T, typename TC>
__global__ void __launch_bounds__(THREADS)
grouped_gemm_kernel(const T* __restrict__ A, long long lda, int gather_div, const int* __restrict__ slot_src,
                    const int* __restrict__ tile_expert, const int* __restrict__ meta, const T* __restrict__ W,
                    long long ldw, long long w_expert, TC* __restrict__ C, long long ldc, int N, int K, int act) {
  __shared__ float As[BK][TILE + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int src_s[TILE];
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  const T* We = W + (size_t)tile_expert[tile] * w_expert;
  if (tid < TILE) src_s[tid] = slot_src[tile * TILE + tid];
  __syncthreads();
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int ty = tid >> 4, tx = tid & 15;
  const int src = src_s[lrow];
  const bool a_ok = src >= 0, w_ok = n0 + lrow < N;
  const T* a_row = A + (size_t)(a_ok ? (gather_div > 0 ? src / gather_div : tile * TILE + lrow) : 0) * lda;
  const T* w_row = We + (size_t)(w_ok ? n0 + lrow : 0) * ldw;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float av[4], wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      av[i] = (a_ok && k < K) ? to_f32(a_row[k]) : 0.f;
      wv[i] = (w_ok && k < K) ? to_f32(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = av[i];
      Ws[lk + i][lrow] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * TM]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * TN]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (src_s[r] < 0) continue;
    TC* c_row = C + (size_t)(tile * TILE + r) * ldc;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) c_row[n] = from_f32<TC>(act_of(acc[i][j], act));
    }
  }
}

// four columns per thread where the rows allow 16-byte loads
template <typename T>
__global__ void combine4_kernel(T* __restrict__ out, const float* __restrict__ y, const int* __restrict__ pair_slot,
                                const float* __restrict__ weights, MaybePartial<T> shared, int top, int width, size_t total4) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = width / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    const int c = (int)(i - t * per_row) * 4;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top; ++j) {
      const int slot = pair_slot[t * top + j];
      if (slot < 0) continue;
      const float w = weights[t * top + j];
      const float4 v = *reinterpret_cast<const float4*>(y + (size_t)slot * width + c);
      s[0] = fmaf(w, v.x, s[0]); s[1] = fmaf(w, v.y, s[1]); s[2] = fmaf(w, v.z, s[2]); s[3] = fmaf(w, v.w, s[3]);
    }
    if (shared.present()) {
#pragma unroll
      for (int k = 0; k < 4; ++k) s[k] += shared.at(t * width + c + k);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) out[t * width + c + k] = from_f32<T>(s[k]);
  }
}

template <typename T>
__global__ void combine_kernel(T* __restrict__ out, const float* __restrict__ y, const int* __restrict__ pair_slot,
                               const float* __restrict__ weights, MaybePartial<T> shared, int top, int width, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    float s = 0.f;
    for (int j = 0; j < top; ++j) {
      const int slot = pair_slot[t * top + j];
      if (slot >= 0) s = fmaf(weights[t * top + j], y[(size_t)slot * width + c], s);
    }
    if (shared.present()) s += shared.at(i);
    out[i] = from_f32<T>(s);
  }
}

}  // namespace

LLMK_API int llmk_moe_tile() { return TILE; }

// logits float32 [n_tokens, experts], or the partial results [splits][n_tokens][experts] of the product that
// makes them; bias float32 [experts] or null; ids int32 [n_tokens, top], weights float32 [n_tokens, top], both in
// the order of falling logits.  over_all: the weights are the chosen experts' shares of the softmax over all experts.
LLMK_API int llmk_moe_topk(const float* logits, const float* partials, int splits, long long split_stride, const float* bias,
                           int* ids, float* weights, int n_tokens, int experts, int top, int over_all, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE((logits != nullptr) != (partials != nullptr), "moe_topk: give logits or partials");
  LLMK_REQUIRE(experts > 0 && experts <= MAX_EXPERTS, "moe_topk: %d experts (1 to %d)", experts, MAX_EXPERTS);
  LLMK_REQUIRE(top > 0 && top <= experts, "moe_topk: top %d of %d experts", top, experts);
  MaybePartial<float> z{logits, partials, splits, split_stride};
  launch_kernel(topk_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream, z, bias, ids,
                weights, n_tokens, experts, top, over_all);
  LLMK_LAUNCH_CHECK("moe_topk");
}

// The sigmoid router with groups (see topk_sigmoid_kernel): correction float32 [experts] or null; groups divides experts;
// 1 <= keep <= groups.
LLMK_API int llmk_moe_topk_sigmoid(const float* logits, const float* partials, int splits, long long split_stride,
                                   const float* correction, int* ids, float* weights, int n_tokens, int experts, int top,
                                   int groups, int keep, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE((logits != nullptr) != (partials != nullptr), "moe_topk_sigmoid: give logits or partials");
  LLMK_REQUIRE(experts > 0 && experts <= MAX_EXPERTS, "moe_topk_sigmoid: %d experts (1 to %d)", experts, MAX_EXPERTS);
  LLMK_REQUIRE(top > 0 && top <= experts, "moe_topk_sigmoid: top %d of %d experts", top, experts);
  LLMK_REQUIRE(groups > 0 && experts % groups == 0 && keep > 0 && keep <= groups,
               "moe_topk_sigmoid: %d experts in %d groups of which %d are kept", experts, groups, keep);
  MaybePartial<float> z{logits, partials, splits, split_stride};
  launch_kernel(topk_sigmoid_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream, z,
                correction, ids, weights, n_tokens, experts, top, groups, keep);
  LLMK_LAUNCH_CHECK("moe_topk_sigmoid");
}

// ids [n_pairs] -> meta[0] (tiles in use), tile_expert [max_tiles], slot_src [max_tiles * 64] (the pair of
// a slot, -1 for padding), pair_slot [n_pairs].  max_tiles >= ceil(n_pairs / 64) + min(experts, n_pairs).
// tile: slots per tile (64 for the CUDA-core products of this file, 128 for the tensor-core ones).
LLMK_API int llmk_moe_group(const int* ids, int n_pairs, int experts, int* meta, int* tile_expert, int* slot_src,
                            int* pair_slot, int max_tiles, int tile, cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  LLMK_REQUIRE(experts > 0 && experts <= MAX_EXPERTS, "moe_group: %d experts (1 to %d)", experts, MAX_EXPERTS);
  LLMK_REQUIRE(tile > 0, "moe_group: tile %d", tile);
  launch_kernel(group_kernel, dim3(1), dim3(1024), 0, stream, ids, n_pairs, experts, meta, tile_expert, slot_src, pair_slot,
                max_tiles, tile);
  LLMK_LAUNCH_CHECK("moe_group");
}

// out [max_tiles * tile, cols] = the rows x[pair / div] in slot order, zeros in padding slots; slots of
// tiles that are not in use are left alone.
LLMK_API int llmk_moe_gather(void* out, const void* x, long long x_stride, const int* slot_src, const int* meta, int div,
                             int cols, int tile, int max_tiles, int dtype, cudaStream_t stream) {
  if (max_tiles == 0 || cols == 0) return 0;
  LLMK_REQUIRE(div > 0 && tile > 0, "moe_gather: bad div %d or tile %d", div, tile);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(gather_rows_by_slot_kernel<T>, dim3((unsigned)(max_tiles * tile)), dim3(128), 0, stream, (T*)out, (const T*)x,
                  x_stride, slot_src, meta, div, cols, tile);
    LLMK_LAUNCH_CHECK("moe_gather");
  });
}

// out_dtype: element kind of C (float32, or the input kind).  act: -1 none, else as llmk_act_rows.
LLMK_API int llmk_moe_gemm(const void* A, long long lda, int gather_div, const int* slot_src, const int* tile_expert,
                           const int* meta, const void* W, long long ldw, long long w_expert, void* C, long long ldc,
                           int N, int K, int max_tiles, int act, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  LLMK_REQUIRE(K > 0 && lda >= K && ldw >= K && ldc >= N, "moe_gemm: bad sizes N=%d K=%d", N, K);
  LLMK_REQUIRE(max_tiles <= 65535, "moe_gemm: %d tiles exceed the grid limit", max_tiles);
  dim3 grid((N + BN - 1) / BN, max_tiles);
#define LLMK_MOE_GEMM(T, TC)                                                                                        \
  launch_kernel(grouped_gemm_kernel<T, TC>, grid, dim3(THREADS), 0, stream, (const T*)A, lda, gather_div, slot_src, \
                tile_expert, meta, (const T*)W, ldw, w_expert, (TC*)C, ldc, N, K, act)
  if (in_dtype == LLMK_F32 && out_dtype == LLMK_F32) LLMK_MOE_GEMM(float, float);
  else if (in_dtype == LLMK_BF16 && out_dtype == LLMK_BF16) LLMK_MOE_GEMM(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LLMK_BF16 && out_dtype == LLMK_F32) LLMK_MOE_GEMM(__nv_bfloat16, float);
  else return llmk_fail(-1, "moe_gemm: unsupported element kinds in=%d out=%d", in_dtype, out_dtype);
#undef LLMK_MOE_GEMM
  LLMK_LAUNCH_CHECK("moe_gemm");
}

// out [n_tokens, width] of the element kind = shared (a tensor, partial results, or nothing) + the
// weighted sum of the pairs' rows of y (float32 [slots, width]).
LLMK_API int llmk_moe_combine(void* out, const float* y, const int* pair_slot, const float* weights, const void* shared,
                              const float* partials, int splits, long long split_stride, int n_tokens, int top, int width,
                              int dtype, cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * width;
  if (total == 0) return 0;
  LLMK_REQUIRE(!(shared && partials), "moe_combine: give shared or partials, not both");
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)llmk_sm_count() * 16) blocks = (size_t)llmk_sm_count() * 16;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> s{(const T*)shared, partials, splits, split_stride};
    if (width % 4 == 0 && (uintptr_t)y % 16 == 0) {
      size_t b4 = (total / 4 + 255) / 256;
      if (b4 > (size_t)llmk_sm_count() * 16) b4 = (size_t)llmk_sm_count() * 16;
      launch_kernel(combine4_kernel<T>, dim3((unsigned)b4), dim3(256), 0, stream, (T*)out, y, pair_slot, weights, s, top, width, total / 4);
    } else {
      launch_kernel(combine_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)out, y, pair_slot, weights, s, top, width, total);
    }
    LLMK_LAUNCH_CHECK("moe_combine");
  });
}
