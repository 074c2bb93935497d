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
// The columns of S never mix: S^T k, the update and S^T q are all per column, and the read-out is taken from the decayed
// state before the write, o = g S^T q + u (k . q), so that both sums over the rows run side by side.  A warp owns eight
// columns of one head: its lanes are 8 row lanes x 4 column lanes, a lane keeps R consecutive rows of two columns in
// registers (R = a head's rows / 8, rounded up to 4, 8, 16 or 32), so a sum over the rows is R multiply-adds in a lane and
// three exchanges between the eight row lanes.  A CTA is WARPS warps (32 columns); its tokens are staged CHUNK at a time:
// the warps norm q and k into shared memory (a row lane's rows lie R + 4 floats apart there, which keeps the eight lanes'
// 16-byte loads on different banks), then every warp walks the chunk on its own, with the next chunk's loads already in
// flight.  (Two-wide float32 multiply-adds on a lane's two columns were tried: fewer instructions, but 927 us against 733 us
// for 2,048 tokens of 8 heads of 128 x 128: the walk is bound by the latency of its dependent steps, not by issue slots.)  The transition of a token is not
// diagonal, so a prompt is not cut into segments here: an entry's tokens run one after another in every CTA of its heads.
#include "common.cuh"

namespace {

#ifndef DELTA_UNROLL
#define DELTA_UNROLL 1
#endif
constexpr int WALK_UNROLL = DELTA_UNROLL;      // tokens of the walk that the compiler may interleave
constexpr int COLS = 2, ROW_LANES = 8, COL_LANES = 4, WARPS = 4, CHUNK = 16, VT = COLS * COL_LANES * WARPS;

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
  constexpr int PITCH = R + 4, DP = ROW_LANES * PITCH;      // floats of one token's q (or k) in shared memory
  constexpr int PER = (ROW_LANES * R + 31) / 32;            // channels a lane stages of a token
  float* q_s = smem;                       // [CHUNK][DP]
  float* k_s = q_s + CHUNK * DP;           // [CHUNK][DP]
  float* v_s = k_s + CHUNK * DP;           // [CHUNK][VT]
  float* o_s = v_s + CHUNK * VT;           // [CHUNK][VT]
  float* g_s = o_s + CHUNK * VT;           // [CHUNK] decay, [CHUNK] beta, [CHUNK] k . q
  float* beta_s = g_s + CHUNK;
  float* kq_s = beta_s + CHUNK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int rl = lane & (ROW_LANES - 1), cl = lane >> 3;
  const int entry = blockIdx.z, head = blockIdx.y;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int dim = a.dim, vdim = a.vdim;
  const int wcol = warp * (COLS * COL_LANES) + cl * COLS;       // the lane's first column within the CTA's VT
  const int col0 = blockIdx.x * VT + wcol;
  const int t0 = a.cu_tokens[entry], t1 = a.cu_tokens[entry + 1];
  if (t0 >= t1) return;
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v, *pb = (const T*)a.b, *pa = (const T*)a.a;
  float* S_g = a.state + (size_t)a.state_slots[entry] * a.slot_stride + ((size_t)head * dim) * vdim;
  const float neg_a = -expf(a.a_log[head]), dt_b = a.dt_bias[head];

  float S[R][COLS];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = rl * R + i;
#pragma unroll
    for (int c = 0; c < COLS; ++c) S[i][c] = (d < dim && col0 + c < vdim) ? S_g[(size_t)d * vdim + col0 + c] : 0.f;
  }

  // What a thread brings of a chunk, requested one chunk ahead so that the loads land under the previous chunk's walk:
  // its warp's tokens (warp, warp + WARPS, ...) of q and k, PER channels a lane; lane j's b and a of the warp's j-th token;
  // and its share of the chunk's values.
  constexpr int TOK = CHUNK / WARPS, VREGS = CHUNK * VT / (WARPS * 32);
  T q_r[TOK][PER], k_r[TOK][PER], v_r[VREGS], b_r = T(), a_r = T();
  auto fetch = [&](int c0) {
    const int n = min(CHUNK, t1 - c0);
#pragma unroll
    for (int j = 0; j < TOK; ++j) {
      const int c = warp + j * WARPS;
      const size_t at = (size_t)(c0 + c) * a.qk_stride + (size_t)qk_head * dim;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (c < n && d < dim) { q_r[j][i] = q[at + d]; k_r[j][i] = k[at + d]; }
      }
    }
    if (lane < TOK && warp + lane * WARPS < n) {
      const size_t ba = (size_t)(c0 + warp + lane * WARPS) * a.ba_stride + head;
      b_r = pb[ba]; a_r = pa[ba];
    }
#pragma unroll
    for (int i = 0; i < VREGS; ++i) {
      const int idx = tid + i * WARPS * 32, cc = blockIdx.x * VT + idx % VT;
      if (idx < n * VT && cc < vdim) v_r[i] = v[(size_t)(c0 + idx / VT) * a.v_stride + (size_t)head * vdim + cc];
    }
  };
  fetch(t0);

  for (int c0 = t0; c0 < t1; c0 += CHUNK) {
    const int n = min(CHUNK, t1 - c0);
    __syncthreads();                         // the previous chunk's outputs have been written out
    // unit q and k of this chunk's tokens, their product, the decay and beta: a warp norms its tokens side by side (the
    // sums of squares and the raw product of all of them go through one round of exchanges)
    {
      float qv[TOK][PER], kv[TOK][PER], red[TOK][3];
#pragma unroll
      for (int j = 0; j < TOK; ++j) {
        const bool live = warp + j * WARPS < n;
        red[j][0] = red[j][1] = red[j][2] = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const bool on = live && lane + 32 * i < dim;
          qv[j][i] = on ? to_f32(q_r[j][i]) : 0.f;
          kv[j][i] = on ? to_f32(k_r[j][i]) : 0.f;
          red[j][0] = fmaf(qv[j][i], qv[j][i], red[j][0]);
          red[j][1] = fmaf(kv[j][i], kv[j][i], red[j][1]);
          red[j][2] = fmaf(qv[j][i], kv[j][i], red[j][2]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int j = 0; j < TOK; ++j)
#pragma unroll
          for (int x = 0; x < 3; ++x) red[j][x] += __shfl_xor_sync(0xffffffffu, red[j][x], o);
#pragma unroll
      for (int j = 0; j < TOK; ++j) {
        const int c = warp + j * WARPS;
        if (c >= n) continue;
        const float rq = a.q_scale / sqrtf(red[j][0] + a.norm_eps), rk = 1.f / sqrtf(red[j][1] + a.norm_eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int d = lane + 32 * i;
          if (d < ROW_LANES * R) {
            q_s[c * DP + (d / R) * PITCH + d % R] = qv[j][i] * rq;
            k_s[c * DP + (d / R) * PITCH + d % R] = kv[j][i] * rk;
          }
        }
        if (lane == j) {
          kq_s[c] = red[j][2] * rq * rk;
          beta_s[c] = 1.f / (1.f + expf(-to_f32(b_r)));
          g_s[c] = expf(neg_a * softplus_d(to_f32(a_r) + dt_b));
        }
      }
    }
#pragma unroll
    for (int i = 0; i < VREGS; ++i) {
      const int idx = tid + i * WARPS * 32;
      if (idx < n * VT) v_s[idx] = blockIdx.x * VT + idx % VT < vdim ? to_f32(v_r[i]) : 0.f;
    }
    __syncthreads();
    if (c0 + CHUNK < t1) fetch(c0 + CHUNK);
#pragma unroll WALK_UNROLL
    for (int c = 0; c < n; ++c) {
      const float g = g_s[c], beta = beta_s[c], kq = kq_s[c];
      float kd[R];
      float pk[COLS][2], pq[COLS][2];          // two partial sums each: the chains of multiply-adds are half as long
#pragma unroll
      for (int cc = 0; cc < COLS; ++cc) pk[cc][0] = pk[cc][1] = pq[cc][0] = pq[cc][1] = 0.f;
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + c * DP + rl * PITCH + i);
        const float4 q4 = *reinterpret_cast<const float4*>(q_s + c * DP + rl * PITCH + i);
        kd[i] = k4.x; kd[i + 1] = k4.y; kd[i + 2] = k4.z; kd[i + 3] = k4.w;
        const float qd[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int cc = 0; cc < COLS; ++cc) {
            pk[cc][j & 1] = fmaf(S[i + j][cc], kd[i + j], pk[cc][j & 1]);
            pq[cc][j & 1] = fmaf(S[i + j][cc], qd[j], pq[cc][j & 1]);
          }
      }
      float sk[COLS], sq[COLS];
#pragma unroll
      for (int cc = 0; cc < COLS; ++cc) { sk[cc] = pk[cc][0] + pk[cc][1]; sq[cc] = pq[cc][0] + pq[cc][1]; }
#pragma unroll
      for (int o = ROW_LANES / 2; o > 0; o >>= 1) {
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          sk[cc] += __shfl_xor_sync(0xffffffffu, sk[cc], o);
          sq[cc] += __shfl_xor_sync(0xffffffffu, sq[cc], o);
        }
      }
      const float2 v2 = *reinterpret_cast<const float2*>(v_s + c * VT + wcol);
      const float vv[COLS] = {v2.x, v2.y};
      float u[COLS], o2[COLS];
#pragma unroll
      for (int cc = 0; cc < COLS; ++cc) {
        u[cc] = beta * (vv[cc] - g * sk[cc]);
        o2[cc] = fmaf(u[cc], kq, g * sq[cc]);
      }
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) S[i][cc] = fmaf(kd[i], u[cc], g * S[i][cc]);
      if (rl == 0) *reinterpret_cast<float2*>(o_s + c * VT + wcol) = make_float2(o2[0], o2[1]);
    }
    __syncthreads();
    for (int idx = tid; idx < n * VT; idx += WARPS * 32) {
      const int c = idx / VT, cc = blockIdx.x * VT + idx % VT;
      if (cc < vdim) a.out[(size_t)(c0 + c) * a.out_stride + (size_t)head * vdim + cc] = o_s[idx];
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = rl * R + i;
    if (d >= dim) continue;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (col0 + c < vdim) S_g[(size_t)d * vdim + col0 + c] = S[i][c];
  }
}

template <typename T, int R>
int launch_delta(const DeltaArgs& a, int n_entries, cudaStream_t stream) {
  const size_t smem = ((size_t)2 * CHUNK * ROW_LANES * (R + 4) + 2 * CHUNK * VT + 3 * CHUNK) * sizeof(float);
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
    if (dim <= 32) return launch_delta<T, 4>(args, n_entries, stream);
    if (dim <= 64) return launch_delta<T, 8>(args, n_entries, stream);
    if (dim <= 128) return launch_delta<T, 16>(args, n_entries, stream);
    return launch_delta<T, 32>(args, n_entries, stream);
  });
}
