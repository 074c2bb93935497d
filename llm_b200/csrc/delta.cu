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

// ---- prompts: the rule chunk by chunk ---------------------------------------------------------------------------
// Within a chunk of CC tokens the rule is linear in the state S_0 that enters the chunk.  With L_t the running sum of
// log g over the chunk's tokens (so that exp(L_t - L_s) is the decay from token s to token t):
//     u_t = beta_t (v_t - exp(L_t) S_0^T k_t - sum_{s<t} exp(L_t - L_s) (k_t . k_s) u_s)
// is a unit lower triangular system (I + A) U = beta V - (beta exp(L) K) S_0 with A_ts = beta_t exp(L_t - L_s) (k_t . k_s), so
//     U = W - Y S_0,   W = (I + A)^-1 (beta V),   Y = (I + A)^-1 (beta exp(L) K)
//     o_t = (exp(L_t) q_t)^T S_0 + sum_{s<=t} B_ts u_s,   B_ts = exp(L_t - L_s) (q_t . k_s)
//     S_C = exp(L_C) S_0 + sum_s (exp(L_C - L_s) k_s) u_s^T
// W, Y, B and the scaled q and k do not depend on the state: delta_prepare makes them for every chunk of the step side by
// side (a CTA per chunk and head: unit norms, the two Gram matrices, forward substitution with a column per thread) and
// leaves them chunk by chunk, padded with zeros to whole chunks, Y and the scaled q with the tokens innermost.
// delta_chunk_walk then runs an entry's chunks one after another: per chunk three small matrix products on the CUDA cores
// with the operands in shared memory (asynchronous copies, the next chunk's under this chunk's arithmetic) and register
// tiles of 16 to 32 sums a thread, the state's tile in registers from chunk to chunk and mirrored in shared memory for the
// products that read all of it.  What is left of the chain from token to token is one step per chunk.  All of it float32;
// the sums of a token are grouped by where its chunk begins, which moves results by rounding only.
constexpr int CC = 32;

struct PrepArgs {
  const void *q, *k; long long qk_stride;
  const void* v; long long v_stride;
  const void *b, *a; long long ba_stride;
  const float *a_log, *dt_bias;
  const int* cu_tokens; int n_entries;
  int heads, qk_heads, dim, vdim;
  float q_scale, norm_eps;
  // per chunk c and head h, at (c * heads + h) * size: YQ [dim][2 CC] (Y's tokens, then the scaled q's), K [CC][dim],
  // W [CC][vdim], B [CC][CC], G [1] (the chunk's whole decay)
  float *YQ, *K, *W, *B, *G;
};

// The chunk with the running number idx: its first token and its length, or false when the step has fewer chunks.
__device__ __forceinline__ bool chunk_of(const int* cu_tokens, int n_entries, int idx, int& c0, int& n) {
  for (int e = 0; e < n_entries; ++e) {
    const int t0 = cu_tokens[e], len = cu_tokens[e + 1] - t0, chunks = (len + CC - 1) / CC;
    if (idx < chunks) { c0 = t0 + idx * CC; n = min(CC, len - idx * CC); return true; }
    idx -= chunks;
  }
  return false;
}

template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(PrepArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  int c0, n;
  if (!chunk_of(a.cu_tokens, a.n_entries, blockIdx.x, c0, n)) return;
  const int head = blockIdx.y, qk_head = head / (a.heads / a.qk_heads);
  const int dim = a.dim, vdim = a.vdim, pitch = dim + 1;
  const size_t unit = (size_t)blockIdx.x * a.heads + head;
  float* kn = smem;                        // [CC][dim + 1]
  float* qn = kn + CC * pitch;             // [CC][dim + 1]
  float* A_s = qn + CC * pitch;            // [CC][CC + 1]
  float* beta_s = A_s + CC * (CC + 1);     // [CC]
  float* L_s = beta_s + CC;                // [CC]: log g, then its running sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v, *pb = (const T*)a.b, *pa = (const T*)a.a;
  const float neg_a = -expf(a.a_log[head]), dt_b = a.dt_bias[head];
  // unit q and k, beta and log g: a warp per token
  for (int t = warp; t < CC; t += 8) {
    const size_t at = (size_t)(c0 + t) * a.qk_stride + (size_t)qk_head * dim;
    float sq = 0.f, sk = 0.f;
    if (t < n)
      for (int d = lane; d < dim; d += 32) {
        const float x = to_f32(q[at + d]), y = to_f32(k[at + d]);
        sq = fmaf(x, x, sq); sk = fmaf(y, y, sk);
      }
    const float rq = a.q_scale / sqrtf(warp_sum(sq) + a.norm_eps), rk = 1.f / sqrtf(warp_sum(sk) + a.norm_eps);
    for (int d = lane; d < dim; d += 32) {
      qn[t * pitch + d] = t < n ? to_f32(q[at + d]) * rq : 0.f;
      kn[t * pitch + d] = t < n ? to_f32(k[at + d]) * rk : 0.f;
    }
    if (lane == 0) {
      const size_t ba = (size_t)(c0 + t) * a.ba_stride + head;
      beta_s[t] = t < n ? 1.f / (1.f + expf(-to_f32(pb[ba]))) : 0.f;
      L_s[t] = t < n ? neg_a * softplus_d(to_f32(pa[ba]) + dt_b) : 0.f;      // log g: the decay without its exponential
    }
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int t = 0; t < CC; ++t) { run += L_s[t]; L_s[t] = run; }
  }
  __syncthreads();
  // the two Gram matrices with their decays
  for (int idx = tid; idx < CC * CC; idx += 256) {
    const int t = idx / CC, s2 = idx % CC;
    float kk = 0.f, qk = 0.f;
    if (s2 <= t && t < n) {
      for (int d = 0; d < dim; ++d) {
        const float ks = kn[s2 * pitch + d];
        kk = fmaf(kn[t * pitch + d], ks, kk);
        qk = fmaf(qn[t * pitch + d], ks, qk);
      }
      const float e = expf(L_s[t] - L_s[s2]);
      kk *= e * beta_s[t];
      qk *= e;
    }
    A_s[t * (CC + 1) + s2] = s2 < t ? kk : 0.f;
    a.B[unit * CC * CC + idx] = (s2 <= t && t < n) ? qk : 0.f;
  }
  __syncthreads();
  // forward substitution: a thread per column of [beta V | beta exp(L) K], the column in registers
  for (int col = tid; col < vdim + dim; col += 256) {
    float x[CC];
    const bool is_v = col < vdim;
    const int d = col - vdim;
#pragma unroll
    for (int t = 0; t < CC; ++t) {
      float r = 0.f;
      if (t < n)
        r = is_v ? beta_s[t] * to_f32(v[(size_t)(c0 + t) * a.v_stride + (size_t)head * vdim + col])
                 : beta_s[t] * expf(L_s[t]) * kn[t * pitch + d];
      x[t] = r;
    }
#pragma unroll
    for (int t = 1; t < CC; ++t) {
      float r = x[t];
#pragma unroll
      for (int s2 = 0; s2 < t; ++s2) r = fmaf(-A_s[t * (CC + 1) + s2], x[s2], r);
      x[t] = r;
    }
    if (is_v) {
#pragma unroll
      for (int t = 0; t < CC; ++t) a.W[(unit * CC + t) * vdim + col] = x[t];
    } else {                                 // Y with the tokens innermost: the column as it lies in the registers
      float* dst = a.YQ + (unit * dim + d) * (2 * CC);
#pragma unroll
      for (int t = 0; t < CC; t += 4) *reinterpret_cast<float4*>(dst + t) = make_float4(x[t], x[t + 1], x[t + 2], x[t + 3]);
    }
  }
  // q and k with the decays that the walk needs: to the token from the chunk's start, from the token to the chunk's end
  const float L_end = L_s[n - 1];
  for (int idx = tid; idx < CC * dim; idx += 256) {
    const int t = idx % CC, d = idx / CC;
    a.YQ[(unit * dim + d) * (2 * CC) + CC + t] = t < n ? expf(L_s[t]) * qn[t * pitch + d] : 0.f;
  }
  for (int idx = tid; idx < CC * dim; idx += 256) {
    const int t = idx / dim, d = idx % dim;
    a.K[(unit * CC + t) * dim + d] = t < n ? expf(L_end - L_s[t]) * kn[t * pitch + d] : 0.f;
  }
  if (tid == 0) a.G[unit] = expf(L_end);
}

struct WalkArgs {
  float* out; long long out_stride;
  const float *YQ, *K, *W, *B, *G;
  float* state; long long slot_stride;
  const int *state_slots, *cu_tokens;
  int heads, dim, vdim;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int WT = 128, WV = 16;             // threads of a walking CTA, value columns it owns
constexpr int TXN = WV / 4, TYN = WT / TXN;  // the threads as TYN x TXN: a thread's 4 columns start at 4 tx
static_assert(2 * CC % TYN == 0 && CC % TYN == 0, "rows of the products divide among the threads");

// RT: rows of the state a thread keeps (a head's rows / 32, rounded up to 1, 2, 4 or 8).  STAGES chunks of operands lie in
// shared memory (2: the next chunk's copies run under this chunk's arithmetic; 1 where two do not fit).
template <int RT, int STAGES>
__global__ void __launch_bounds__(WT)
delta_chunk_walk_kernel(WalkArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DPAD = TYN * RT, BP = CC + 4, RA = 2 * CC / TYN, RB = CC / TYN;      // rows a thread takes of the two products
  constexpr int STAGE = DPAD * 2 * CC + CC * DPAD + CC * WV + CC * BP;      // floats of one stage: YQ, K, W, B
  float* S_s = smem + STAGES * STAGE;      // [DPAD][WV]: the state as the products read it
  float* u_s = S_s + DPAD * WV;            // [CC][WV]
  float* o_s = u_s + CC * WV;              // [CC][WV]
  const int tid = threadIdx.x, ty = tid / TXN, tx = tid % TXN;
  const int entry = blockIdx.z, head = blockIdx.y;
  const int dim = a.dim, vdim = a.vdim, colb = blockIdx.x * WV;
  const int t0 = a.cu_tokens[entry], t1 = a.cu_tokens[entry + 1];
  if (t0 >= t1) return;
  int chunk = 0;                            // the running number of the entry's first chunk
  for (int e = 0; e < entry; ++e) chunk += (a.cu_tokens[e + 1] - a.cu_tokens[e] + CC - 1) / CC;
  const bool vec = dim % 4 == 0 && vdim % 4 == 0;
  float* S_g = a.state + (size_t)a.state_slots[entry] * a.slot_stride + ((size_t)head * dim) * vdim;
  float S[RT][4];                           // rows RT ty .., columns 4 tx ..
#pragma unroll
  for (int i = 0; i < RT; ++i) {
    const int d = ty * RT + i;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = colb + 4 * tx + c;
      S[i][c] = (d < dim && col < vdim) ? S_g[(size_t)d * vdim + col] : 0.f;
    }
    *reinterpret_cast<float4*>(S_s + d * WV + 4 * tx) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
  }
  // request the operands of chunk number c into a stage (they are padded with zeros to whole chunks where they were made)
  auto issue = [&](int c, float* st) {
    const size_t unit = (size_t)c * a.heads + head;
    float *yq_s = st, *k_s = st + DPAD * 2 * CC, *w_s = k_s + CC * DPAD, *b_s = w_s + CC * WV;
    if (vec) {
      const float* src = a.YQ + unit * dim * 2 * CC;
      for (int i = tid; i < dim * 2 * CC / 4; i += WT) cp_async16(yq_s + 4 * i, src + 4 * i);
      src = a.K + unit * CC * dim;
      for (int i = tid; i < CC * dim / 4; i += WT) { const int t = (4 * i) / dim, d = (4 * i) % dim; cp_async16(k_s + t * DPAD + d, src + 4 * i); }
      src = a.W + unit * CC * vdim;
      for (int i = tid; i < CC * WV / 4; i += WT) {
        const int t = (4 * i) / WV, c4 = (4 * i) % WV;
        if (colb + c4 < vdim) cp_async16(w_s + 4 * i, src + (size_t)t * vdim + colb + c4);
      }
    } else {
      const float* src = a.YQ + unit * dim * 2 * CC;
      for (int i = tid; i < dim * 2 * CC; i += WT) yq_s[i] = src[i];
      src = a.K + unit * CC * dim;
      for (int i = tid; i < CC * dim; i += WT) k_s[(i / dim) * DPAD + i % dim] = src[i];
      src = a.W + unit * CC * vdim;
      for (int i = tid; i < CC * WV; i += WT) if (colb + i % WV < vdim) w_s[i] = src[(size_t)(i / WV) * vdim + colb + i % WV];
    }
    const float* src = a.B + unit * CC * CC;
    for (int i = tid; i < CC * CC / 4; i += WT) cp_async16(b_s + ((4 * i) / CC) * BP + (4 * i) % CC, src + 4 * i);
    cp_async_commit();
  };
  // rows of K beyond the head's and columns of W beyond the values' are never copied: they stay zero
  for (int i = tid; i < STAGES * STAGE; i += WT) smem[i] = 0.f;
  __syncthreads();
  issue(chunk, smem);
  int at_stage = 0;
  for (int c0 = t0; c0 < t1; c0 += CC, ++chunk) {
    const int n = min(CC, t1 - c0);
    const float g_end = a.G[(size_t)chunk * a.heads + head];
    const float* st = smem + at_stage * STAGE;
    const float *yq_s = st, *k_s = st + DPAD * 2 * CC, *w_s = k_s + CC * DPAD, *b_s = w_s + CC * WV;
    const bool more = c0 + CC < t1;
    if (STAGES == 2 && more) {
      issue(chunk + 1, smem + (at_stage ^ 1) * STAGE);      // that stage's last readers passed the barrier below
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                         // the stage has landed; S_s holds the state that enters the chunk
    // [Y; exp(L) Q] S_0: 2 CC rows x WV columns, a thread RA rows (RA ty ..) x 4 columns
    {
      float acc[RA][4];
#pragma unroll
      for (int i = 0; i < RA; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
      // four rows of the state and of the operands a step, the next step's loads issued before this step's multiply-adds
      // (one warp per scheduler hides nothing by itself); rows beyond the head's are zero on both sides
      float4 sa[4], sb[4];
      float2 ra[4], rb[4];
      auto load = [&](int d0, float4 (&sv)[4], float2 (&rv)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sv[j] = *reinterpret_cast<const float4*>(S_s + (d0 + j) * WV + 4 * tx);
          rv[j] = *reinterpret_cast<const float2*>(yq_s + (d0 + j) * 2 * CC + RA * ty);
        }
      };
      auto mac = [&](const float4 (&sv)[4], const float2 (&rv)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float s4[4] = {sv[j].x, sv[j].y, sv[j].z, sv[j].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            acc[0][c] = fmaf(rv[j].x, s4[c], acc[0][c]);
            acc[1][c] = fmaf(rv[j].y, s4[c], acc[1][c]);
          }
        }
      };
      static_assert(RA == 2 && DPAD % 8 == 0, "a thread takes two rows of [Y; Q]");
      load(0, sa, ra);
#pragma unroll 1
      for (int d0 = 0; d0 < DPAD; d0 += 8) {
        load(d0 + 4, sb, rb);
        mac(sa, ra);
        if (d0 + 8 < DPAD) load(d0 + 8, sa, ra);
        mac(sb, rb);
      }
#pragma unroll
      for (int i = 0; i < RA; ++i) {
        const int row = RA * ty + i;          // < CC: a row of Y (u = w - y S_0); else a row of the scaled q
        if (row < CC) {
          const float4 w4 = *reinterpret_cast<const float4*>(w_s + row * WV + 4 * tx);
          *reinterpret_cast<float4*>(u_s + row * WV + 4 * tx) = make_float4(w4.x - acc[i][0], w4.y - acc[i][1], w4.z - acc[i][2], w4.w - acc[i][3]);
        } else {
          *reinterpret_cast<float4*>(o_s + (row - CC) * WV + 4 * tx) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
      }
    }
    __syncthreads();
    // the outputs: o_t = (state's share) + sum_{s <= t} B_ts u_s; a thread RB tokens (RB ty ..) x 4 columns
    {
      float4 o[RB];
#pragma unroll
      for (int i = 0; i < RB; ++i) o[i] = *reinterpret_cast<const float4*>(o_s + (RB * ty + i) * WV + 4 * tx);
#pragma unroll 8
      for (int s2 = 0; s2 < CC; ++s2) {      // B is zero beyond the diagonal
        const float4 u4 = *reinterpret_cast<const float4*>(u_s + s2 * WV + 4 * tx);
#pragma unroll
        for (int i = 0; i < RB; ++i) {
          const float bts = b_s[(RB * ty + i) * BP + s2];
          o[i].x = fmaf(bts, u4.x, o[i].x); o[i].y = fmaf(bts, u4.y, o[i].y);
          o[i].z = fmaf(bts, u4.z, o[i].z); o[i].w = fmaf(bts, u4.w, o[i].w);
        }
      }
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int t = RB * ty + i, col = colb + 4 * tx;
        if (t >= n) continue;
        float* dst = a.out + (size_t)(c0 + t) * a.out_stride + (size_t)head * vdim + col;
        const float ov[4] = {o[i].x, o[i].y, o[i].z, o[i].w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (col + c < vdim) dst[c] = ov[c];
      }
    }
    // the state at the chunk's end: exp(L_C) S_0 + (scaled K)^T U; a thread RT rows x 4 columns, kept in registers
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) S[i][c] *= g_end;
    {
      float4 ua, ub;
      float ka[RT], kb[RT];
      auto load = [&](int s2, float4& u4, float (&kv)[RT]) {
        u4 = *reinterpret_cast<const float4*>(u_s + s2 * WV + 4 * tx);
        const float* kr = k_s + s2 * DPAD + ty * RT;
        if (RT % 4 == 0) {
#pragma unroll
          for (int i = 0; i < RT; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
            kv[i] = k4.x; kv[(i + 1) % RT] = k4.y; kv[(i + 2) % RT] = k4.z; kv[(i + 3) % RT] = k4.w;      // (the wrap only quiets the bounds check where RT < 4)
          }
        } else {
#pragma unroll
          for (int i = 0; i < RT; ++i) kv[i] = kr[i];
        }
      };
      auto mac = [&](const float4& u4, const float (&kv)[RT]) {
        const float uv[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < RT; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) S[i][c] = fmaf(kv[i], uv[c], S[i][c]);
      };
      load(0, ua, ka);
#pragma unroll 2
      for (int s2 = 0; s2 < CC; s2 += 2) {
        load(s2 + 1, ub, kb);
        mac(ua, ka);
        if (s2 + 2 < CC) load(s2 + 2, ua, ka);
        mac(ub, kb);
      }
    }
    __syncthreads();                         // every thread is done with this stage, u_s, o_s and the old S_s
#pragma unroll
    for (int i = 0; i < RT; ++i)
      *reinterpret_cast<float4*>(S_s + (ty * RT + i) * WV + 4 * tx) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
    if (STAGES == 2) at_stage ^= 1;
    else if (more) issue(chunk + 1, smem);
  }
#pragma unroll
  for (int i = 0; i < RT; ++i) {
    const int d = ty * RT + i;
    if (d >= dim) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = colb + 4 * tx + c;
      if (col < vdim) S_g[(size_t)d * vdim + col] = S[i][c];
    }
  }
}

template <int RT>
int launch_walk(const WalkArgs& a, int n_entries, cudaStream_t stream) {
  constexpr int STAGES = RT <= 4 ? 2 : 1;      // two stages of a head of 256 rows exceed an SM's shared memory
  constexpr int DPAD = TYN * RT;
  const size_t stage = (size_t)DPAD * 2 * CC + CC * DPAD + CC * WV + CC * (CC + 4);
  const size_t smem = (STAGES * stage + DPAD * WV + 2 * CC * WV) * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(delta_chunk_walk_kernel<RT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_kernel(delta_chunk_walk_kernel<RT, STAGES>, dim3((a.vdim + WV - 1) / WV, a.heads, n_entries), dim3(WT), smem, stream, a);
  LLMK_LAUNCH_CHECK("delta_chunk_walk");
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

// The same rule for a step with prompt portions, chunk by chunk (see delta_prepare_kernel).  n_tokens: the step's tokens.
// Float32 scratch for n_tokens / 32 + n_entries chunks of every head: YQ (dim * 64 floats a chunk and head), K (32 * dim),
// W (32 * vdim), B (32 * 32), G (1).
LLMK_API int llmk_delta_chunk_scan(float* out, long long out_stride, const void* q, const void* k, long long qk_stride,
                                   const void* v, long long v_stride, const void* b, const void* a, long long ba_stride,
                                   const float* a_log, const float* dt_bias, float* state, long long slot_stride,
                                   const int* state_slots, const int* cu_tokens, int n_entries, int n_tokens, int heads,
                                   int qk_heads, int dim, int vdim, float q_scale, float norm_eps, float* YQ, float* K, float* W,
                                   float* B, float* G, int dtype, cudaStream_t stream) {
  if (n_entries == 0 || n_tokens == 0) return 0;
  LLMK_REQUIRE(dim > 0 && dim <= 256, "delta_chunk_scan: key size %d (1 to 256)", dim);
  LLMK_REQUIRE(qk_heads > 0 && heads % qk_heads == 0 && vdim > 0, "delta_chunk_scan: %d heads do not divide into %d key heads", heads, qk_heads);
  LLMK_REQUIRE(n_entries <= 65535 && heads <= 65535, "delta_chunk_scan: too many entries or heads for one launch");
  LLMK_REQUIRE(YQ && K && W && B && G, "delta_chunk_scan: the scratch is missing");
  PrepArgs p = {q, k, qk_stride, v, v_stride, b, a, ba_stride, a_log, dt_bias, cu_tokens, n_entries, heads, qk_heads, dim, vdim,
                q_scale, norm_eps, YQ, K, W, B, G};
  const int chunks = n_tokens / CC + n_entries;
  const size_t smem = ((size_t)2 * CC * (dim + 1) + CC * (CC + 1) + 2 * CC) * sizeof(float);
  int rc = dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(delta_prepare_kernel<T>, dim3(chunks, heads), dim3(256), smem, stream, p);
    LLMK_LAUNCH_CHECK("delta_prepare");
  });
  if (rc) return rc;
  WalkArgs w = {out, out_stride, YQ, K, W, B, G, state, slot_stride, state_slots, cu_tokens, heads, dim, vdim};
  if (dim <= 32) return launch_walk<1>(w, n_entries, stream);
  if (dim <= 64) return launch_walk<2>(w, n_entries, stream);
  if (dim <= 128) return launch_walk<4>(w, n_entries, stream);
  return launch_walk<8>(w, n_entries, stream);
}
