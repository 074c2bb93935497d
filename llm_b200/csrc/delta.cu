// The gated delta rule: a recurrent mixer whose matrix state per head is decayed, corrected toward the new value along the
// new key, and read out, token by token:
//
//   S <- g_t S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t         S [dim, vdim] per head
//   q_t, k_t unit vectors per head (x / sqrt(sum(x^2) + 1e-6)), q_t also times q_scale;
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log) softplus(a_t + dt_bias))                   one number per head and token
//
// Head h reads q/k head h / (heads / qk_heads).  The state is float32 and lives in the request's state slot (zero at
// admission); it is read at the start of an entry's tokens and written back at their end, so a whole prompt, a portion and a
// single token run the same arithmetic, in the same order, whatever else is in the batch.  Norms, beta, the decay, the
// state and every sum are float32; q, k, v, a, b are read in the projections' kind.
//
// The columns of S never mix: S^T k, the update and S^T q are all per column.  So a warp owns COLS columns of one head and
// lane l keeps rows l, l + 32, ... of them in registers; the two products over the rows are warp sums, and the read-out is
// taken from the decayed state before the write, o = g S^T q + u (k . q), so that both sums run side by side.  A CTA is
// WARPS warps (WARPS * COLS columns); its tokens are staged CHUNK at a time: the warps norm q and k into shared memory, then
// every warp walks the chunk on its own.  The transition of a token is not diagonal, so a prompt is not cut into segments
// here: an entry's tokens run one after another in every CTA of its heads.
#include "common.cuh"

namespace {

constexpr int COLS = 4, WARPS = 8, CHUNK = 16, VT = COLS * WARPS;

__device__ __forceinline__ float softplus_d(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaArgs {
  float* out; long long out_stride;                       // [T, heads * vdim] float32
  const void *q, *k; long long qk_stride;                 // [T, qk_heads * dim]
  const void* v; long long v_stride;                      // [T, heads * vdim]
  const void *b, *a; long long ba_stride;                 // [T, heads] each
  const float *a_log, *dt_bias;                           // [heads]
  float* state; long long slot_stride;                    // slot s at state + s * slot_stride: [heads, dim, vdim]
  const int *state_slots, *cu_tokens;
  int heads, qk_heads, dim, vdim;
  float q_scale, norm_eps;
};

template <typename T, int R>
__global__ void __launch_bounds__(WARPS * 32)
delta_scan_kernel(DeltaArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DPAD = 32 * R;
  float* q_s = smem;                       // [CHUNK][DPAD]
  float* k_s = q_s + CHUNK * DPAD;         // [CHUNK][DPAD]
  float* v_s = k_s + CHUNK * DPAD;         // [CHUNK][VT]
  float* o_s = v_s + CHUNK * VT;           // [CHUNK][VT]
  float* g_s = o_s + CHUNK * VT;           // [CHUNK] decay, [CHUNK] beta, [CHUNK] k . q
  float* beta_s = g_s + CHUNK;
  float* kq_s = beta_s + CHUNK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int entry = blockIdx.z, head = blockIdx.y;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int dim = a.dim, vdim = a.vdim;
  const int col0 = blockIdx.x * VT + warp * COLS;
  const int t0 = a.cu_tokens[entry], t1 = a.cu_tokens[entry + 1];
  if (t0 >= t1) return;
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v, *pb = (const T*)a.b, *pa = (const T*)a.a;
  float* S_g = a.state + (size_t)a.state_slots[entry] * a.slot_stride + ((size_t)head * dim) * vdim;
  const float neg_a = -expf(a.a_log[head]), dt_b = a.dt_bias[head];

  float S[R][COLS];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < COLS; ++c) S[i][c] = (d < dim && col0 + c < vdim) ? S_g[(size_t)d * vdim + col0 + c] : 0.f;
  }

  for (int c0 = t0; c0 < t1; c0 += CHUNK) {
    const int n = min(CHUNK, t1 - c0);
    __syncthreads();                         // the previous chunk's outputs have been written out
    // unit q and k of this chunk's tokens, their product, the decay and beta: a warp per token
    for (int c = warp; c < n; c += WARPS) {
      const size_t at = (size_t)(c0 + c) * a.qk_stride + (size_t)qk_head * dim;
      float qv[R], kv[R], sq = 0.f, sk = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < dim ? to_f32(q[at + d]) : 0.f;
        kv[i] = d < dim ? to_f32(k[at + d]) : 0.f;
        sq = fmaf(qv[i], qv[i], sq);
        sk = fmaf(kv[i], kv[i], sk);
      }
      const float rq = a.q_scale / sqrtf(warp_sum(sq) + a.norm_eps), rk = 1.f / sqrtf(warp_sum(sk) + a.norm_eps);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        qv[i] *= rq; kv[i] *= rk;
        q_s[c * DPAD + lane + 32 * i] = qv[i];
        k_s[c * DPAD + lane + 32 * i] = kv[i];
        dot = fmaf(qv[i], kv[i], dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) {
        const size_t ba = (size_t)(c0 + c) * a.ba_stride + head;
        kq_s[c] = dot;
        beta_s[c] = 1.f / (1.f + expf(-to_f32(pb[ba])));
        g_s[c] = expf(neg_a * softplus_d(to_f32(pa[ba]) + dt_b));
      }
    }
    for (int idx = tid; idx < n * VT; idx += WARPS * 32) {
      const int c = idx / VT, cc = blockIdx.x * VT + idx % VT;
      v_s[idx] = cc < vdim ? to_f32(v[(size_t)(c0 + c) * a.v_stride + (size_t)head * vdim + cc]) : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float g = g_s[c], beta = beta_s[c], kq = kq_s[c];
      float kd[R], pk[COLS], pq[COLS];
#pragma unroll
      for (int cc = 0; cc < COLS; ++cc) pk[cc] = pq[cc] = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        kd[i] = k_s[c * DPAD + lane + 32 * i];
        const float qd = q_s[c * DPAD + lane + 32 * i];
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          pk[cc] = fmaf(S[i][cc], kd[i], pk[cc]);
          pq[cc] = fmaf(S[i][cc], qd, pq[cc]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          pk[cc] += __shfl_xor_sync(0xffffffffu, pk[cc], o);
          pq[cc] += __shfl_xor_sync(0xffffffffu, pq[cc], o);
        }
      }
      const float4 v4 = *reinterpret_cast<const float4*>(v_s + c * VT + warp * COLS);
      const float vv[COLS] = {v4.x, v4.y, v4.z, v4.w};
      float u[COLS], o4[COLS];
#pragma unroll
      for (int cc = 0; cc < COLS; ++cc) {
        u[cc] = beta * (vv[cc] - g * pk[cc]);
        o4[cc] = fmaf(u[cc], kq, g * pq[cc]);
      }
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) S[i][cc] = fmaf(kd[i], u[cc], g * S[i][cc]);
      if (lane == 0) *reinterpret_cast<float4*>(o_s + c * VT + warp * COLS) = make_float4(o4[0], o4[1], o4[2], o4[3]);
    }
    __syncthreads();
    for (int idx = tid; idx < n * VT; idx += WARPS * 32) {
      const int c = idx / VT, cc = blockIdx.x * VT + idx % VT;
      if (cc < vdim) a.out[(size_t)(c0 + c) * a.out_stride + (size_t)head * vdim + cc] = o_s[idx];
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = lane + 32 * i;
    if (d >= dim) continue;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (col0 + c < vdim) S_g[(size_t)d * vdim + col0 + c] = S[i][c];
  }
}

template <typename T, int R>
int launch_delta(const DeltaArgs& a, int n_entries, cudaStream_t stream) {
  const size_t smem = ((size_t)2 * CHUNK * 32 * R + 2 * CHUNK * VT + 3 * CHUNK) * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const dim3 grid((a.vdim + VT - 1) / VT, a.heads, n_entries);
  launch_kernel(delta_scan_kernel<T, R>, grid, dim3(WARPS * 32), smem, stream, a);
  LLMK_LAUNCH_CHECK("delta_scan");
}

}  // namespace

// q, k [T, qk_heads * dim] (one row stride), v [T, heads * vdim], b and a [T, heads] (one row stride), all in the
// projections' kind; a_log, dt_bias float32 [heads]; state float32, slot s at state + s * slot_stride holding
// [heads, dim, vdim]; out float32 [T, heads * vdim].  q is scaled by q_scale after its unit norm; norm_eps is added to the
// sums of squares.
LLMK_API int llmk_delta_scan(float* out, long long out_stride, const void* q, const void* k, long long qk_stride, const void* v,
                             long long v_stride, const void* b, const void* a, long long ba_stride, const float* a_log,
                             const float* dt_bias, float* state, long long slot_stride, const int* state_slots,
                             const int* cu_tokens, int n_entries, int heads, int qk_heads, int dim, int vdim, float q_scale,
                             float norm_eps, int dtype, cudaStream_t stream) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(dim > 0 && dim <= 256, "delta_scan: key size %d (1 to 256)", dim);
  LLMK_REQUIRE(qk_heads > 0 && heads % qk_heads == 0 && vdim > 0, "delta_scan: %d heads do not divide into %d key heads", heads, qk_heads);
  LLMK_REQUIRE(n_entries <= 65535 && heads <= 65535, "delta_scan: too many entries or heads for one launch");
  DeltaArgs args = {out, out_stride, q, k, qk_stride, v, v_stride, b, a, ba_stride, a_log, dt_bias, state, slot_stride,
                    state_slots, cu_tokens, heads, qk_heads, dim, vdim, q_scale, norm_eps};
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    if (dim <= 32) return launch_delta<T, 1>(args, n_entries, stream);
    if (dim <= 64) return launch_delta<T, 2>(args, n_entries, stream);
    if (dim <= 128) return launch_delta<T, 4>(args, n_entries, stream);
    return launch_delta<T, 8>(args, n_entries, stream);
  });
}
