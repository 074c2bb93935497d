// Recurrent mixers with a matrix state per head and a diagonal decay, beside the gated linear attention of recurrent.cu:
//
//   bonus form (RWKV-style time mixing):   o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T
//                                          w_t = exp(-exp(z_t + w0))   per head and key channel
//   scalar form (state-space duality):     S_t = a_t S_{t-1} + dt_t B_t x_t^T,          y_t = S_t^T C_t + D x_t
//                                          dt_t = softplus(dt'_t + dt_bias),  a_t = exp(-exp(A_log) dt_t)   per head;
//                                          B and C are shared by the heads of a group
//   gate form (HGRN2):                     S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,   o_t = S_t^T silu(q_t)
//                                          f_t = l + (1 - l) sigmoid(z_t + b)   per head and key channel, l a lower bound:
//                                          what the forget gate lets go is what is written, so there is no key
//
// S [dim, vdim] is float32 and lives in the request's state slot (zero at admission); it is read at the start of an
// entry's tokens and written back at their end, so prompts, portions and single tokens run the same arithmetic.  Decays,
// their logarithms, step sizes, state and sums are float32; r, k, v (x, B, C, dt') are read in the projections' kind.
//
// Work split as in recurrent.cu: a CTA owns (entry, head, VT value columns); thread (j, g) keeps the 8 x 4 block of S at
// rows 8 g .., columns 4 j .. in registers; tokens are staged in shared memory CHUNK at a time; the partial outputs of the
// row groups are summed in the order of g.
//
// Long entries (prompts) run as segments of seg_len tokens side by side, as in recurrent.cu: pass 1 walks every segment but
// an entry's last from a zero state and leaves its end state and the product of its decays; a chain kernel turns those into
// every segment's true start state (start_(s+1) = diag(P_s) start_s + E_s, from the request's state); pass 2 walks every
// segment from its true start, writes the outputs, and the entry's last segment writes the request's state.  The float32
// sums of a token's state are then grouped by where its segment begins, which moves results by rounding only.
//
// Also here: the token shift that feeds the bonus form's projections, the gated RMS norm over groups of channels that
// follows either form, and the mean of two normed rows (two mixers side by side).
#include "common.cuh"

namespace {

constexpr int ROWS = 8, COLS = 4, CHUNK = 8, MAX_GROUPS = 32;
enum : int { FORM_BONUS = 0, FORM_SCALAR = 1, FORM_GATE = 2 };

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct ScanArgs {
  float* out; long long out_stride;              // [T, heads * vdim] float32
  const void *q, *k, *v; long long qk_stride, v_stride;      // q, k: [T, qk_heads * dim]; v: [T, heads * vdim]
  const float* z; long long z_stride;            // bonus form: the decay's pre-activation [T, heads * dim] float32
  const float* z_bias;                           // bonus form: w0 [heads * dim]
  const float* bonus;                            // bonus form: u [heads, dim]; gate form: the lower bound l [heads, dim]
  const void* dt; long long dt_stride;           // scalar form: dt' [T, heads]
  const float *dt_bias, *a_log, *skip;           // scalar form: [heads] each
  float* state; long long slot_stride;           // slot s at state + s * slot_stride: [heads, dim, vdim]
  const int *state_slots, *cu_tokens;
  int heads, qk_heads, dim, vdim;
  // bonus form: the last input row of every entry is kept for the next step's token shift
  const void* shift_src; long long shift_stride; float* shift_state; long long shift_slot_stride; int shift_width;
  // segments: seg_len 0 = one pass over the whole entry (mode 0); else mode 1 or 2 (the two passes), at most max_segs
  // segments per entry, seg_state [segments, heads, dim, vdim] and seg_decay [segments, heads, dim] float32 scratch
  int seg_len, max_segs, mode; float* seg_state; float* seg_decay;
};

// STATE_ONLY: the first pass over segments, which needs end states and decay products but no outputs (no q, no sums).
template <typename T, int VT, int FORM, bool STATE_ONLY>
__global__ void __launch_bounds__(VT / COLS * MAX_GROUPS, 2)
diag_scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int TX = VT / COLS;
  static_assert(TX == ROWS, "a thread stages the channel of its own index: threads per row group = rows per group");
  const int groups = blockDim.y, dpad = groups * ROWS;
  float* q_s = smem;                          // [CHUNK][dpad]
  float* k_s = q_s + CHUNK * dpad;
  float* a_s = k_s + CHUNK * dpad;            // bonus form: [CHUNK][dpad]; scalar form: [CHUNK] (one decay per token)
  float* v_s = a_s + CHUNK * dpad;            // [CHUNK][VT]
  float* part = v_s + CHUNK * VT;             // [CHUNK][groups][VT]
  const int j = threadIdx.x, g = threadIdx.y;
  const int tid = g * TX + j, nthreads = TX * groups;
  const int mode = a.mode;
  const int entry = a.seg_len ? blockIdx.z / a.max_segs : blockIdx.z, head = blockIdx.y;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int col0 = blockIdx.x * VT + j * COLS;
  const int dim = a.dim, vdim = a.vdim;
  int t0 = a.cu_tokens[entry], t1 = a.cu_tokens[entry + 1];
  const int t_end = t1;
  size_t seg_index = 0;
  if (a.seg_len) {
    const int seg = blockIdx.z % a.max_segs;
    if (seg * a.seg_len >= t1 - t0) return;
    for (int e = 0; e < entry; ++e) seg_index += (a.cu_tokens[e + 1] - a.cu_tokens[e] + a.seg_len - 1) / a.seg_len;
    seg_index += seg;
    t0 += seg * a.seg_len;
    t1 = min(t1, t0 + a.seg_len);
    if (mode == 1 && t1 == t_end) return;               // nothing follows an entry's last segment
  }
  const bool last = t1 == t_end;
  const T *q = (const T*)a.q, *k = (const T*)a.k, *v = (const T*)a.v;
  float* S_slot = a.state + (size_t)a.state_slots[entry] * a.slot_stride + ((size_t)head * dim) * vdim;
  float* S_seg = a.seg_state + ((seg_index * a.heads + head) * dim) * vdim;
  float* S_g = mode == 0 ? S_slot : S_seg;

  if (FORM == FORM_BONUS && a.shift_state && blockIdx.x == 0 && head == 0 && t1 > t0 && last && mode != 1) {
    const T* src = (const T*)a.shift_src + (size_t)(t1 - 1) * a.shift_stride;
    float* dst = a.shift_state + (size_t)a.state_slots[entry] * a.shift_slot_stride;
    for (int c = tid; c < a.shift_width; c += nthreads) dst[c] = to_f32(src[c]);
  }

  float S[ROWS][COLS], U[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = g * ROWS + r;
#pragma unroll
    for (int c = 0; c < COLS; ++c) S[r][c] = (mode != 1 && d < dim && col0 + c < vdim) ? S_g[(size_t)d * vdim + col0 + c] : 0.f;
    U[r] = (FORM == FORM_BONUS && d < dim) ? a.bonus[head * dim + d] : 0.f;
  }
  float A[ROWS];                              // pass 1: the product of the segment's decays, per key channel
#pragma unroll
  for (int r = 0; r < ROWS; ++r) A[r] = 1.f;
  const float neg_a = FORM == FORM_SCALAR ? -expf(a.a_log[head]) : 0.f;
  const float skip = FORM == FORM_SCALAR ? a.skip[head] : 0.f;
  const float dt_b = FORM == FORM_SCALAR ? a.dt_bias[head] : 0.f;

  // What a thread brings of a chunk: channel d = tid of every token's q, k (and z), and up to VREGS of its values.  The
  // next chunk's loads are issued before this chunk's multiply-adds and land under them.
  constexpr int VREGS = 8;
  const bool v_regs = CHUNK * VT <= VREGS * nthreads;       // else (fewer than 32 channels) the values are read when staged
  T q_r[CHUNK], k_r[CHUNK], v_r[VREGS], dt_r;
  float z_r[CHUNK];
  const float zb = (FORM != FORM_SCALAR && tid < dim && a.z_bias) ? a.z_bias[head * dim + tid] : 0.f;
  const float low = (FORM == FORM_GATE && tid < dim) ? a.bonus[head * dim + tid] : 0.f;
  auto fetch = [&](int c0) {
    const int n = min(CHUNK, t1 - c0);
#pragma unroll
    for (int c = 0; c < CHUNK; ++c) {
      if (c < n && tid < dim) {
        const size_t at = (size_t)(c0 + c) * a.qk_stride + (size_t)qk_head * dim + tid;
        if (!STATE_ONLY) q_r[c] = q[at];
        if (FORM != FORM_GATE) k_r[c] = k[at];
        if (FORM != FORM_SCALAR) z_r[c] = a.z[(size_t)(c0 + c) * a.z_stride + (size_t)head * dim + tid];
      }
    }
    if (v_regs) {
#pragma unroll
      for (int i = 0; i < VREGS; ++i) {
        const int idx = tid + i * nthreads, cc = blockIdx.x * VT + idx % VT;
        if (idx < n * VT && cc < vdim) v_r[i] = v[(size_t)(c0 + idx / VT) * a.v_stride + (size_t)head * vdim + cc];
      }
    }
    if (FORM == FORM_SCALAR && tid < n) dt_r = ((const T*)a.dt)[(size_t)(c0 + tid) * a.dt_stride + head];
  };
  if (t0 < t1) fetch(t0);

  for (int c0 = t0; c0 < t1; c0 += CHUNK) {
    const int n = min(CHUNK, t1 - c0);
    __syncthreads();                          // the previous chunk's partial sums have been read
    if (FORM == FORM_SCALAR) {
      if (tid < n) a_s[tid] = softplus_f(to_f32(dt_r) + dt_b);
      __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < CHUNK; ++c) {
      if (c >= n) break;
      float qv = 0.f, kv = 0.f, av = 0.f;
      if (tid < dim) {
        if (!STATE_ONLY) qv = to_f32(q_r[c]);
        if (FORM == FORM_GATE) {
          if (!STATE_ONLY) qv = qv / (1.f + expf(-qv));
          av = low + (1.f - low) / (1.f + expf(-(z_r[c] + zb)));
          kv = 1.f - av;
        } else {
          kv = to_f32(k_r[c]);
          if (FORM == FORM_BONUS)
            av = expf(-expf(z_r[c] + zb));
          else
            kv *= a_s[c];                       // dt B
        }
      }
      if (!STATE_ONLY) q_s[c * dpad + tid] = qv;
      k_s[c * dpad + tid] = kv;
      if (FORM != FORM_SCALAR) a_s[c * dpad + tid] = av;
    }
    if (v_regs) {
#pragma unroll
      for (int i = 0; i < VREGS; ++i) {
        const int idx = tid + i * nthreads;
        if (idx < n * VT) v_s[idx] = blockIdx.x * VT + idx % VT < vdim ? to_f32(v_r[i]) : 0.f;
      }
    } else {
      for (int idx = tid; idx < n * VT; idx += nthreads) {
        const int c = idx / VT, jj = idx % VT, cc = blockIdx.x * VT + jj;
        v_s[idx] = cc < vdim ? to_f32(v[(size_t)(c0 + c) * a.v_stride + (size_t)head * vdim + cc]) : 0.f;
      }
    }
    __syncthreads();
    if (c0 + CHUNK < t1) fetch(c0 + CHUNK);
    for (int c = 0; c < n; ++c) {
      const float4 v4 = *reinterpret_cast<const float4*>(v_s + c * VT + j * COLS);
      const float vv[COLS] = {v4.x, v4.y, v4.z, v4.w};
      float kc[ROWS], ac[ROWS], qc[ROWS];
      const float a_tok = FORM == FORM_SCALAR ? expf(neg_a * a_s[c]) : 0.f;
#pragma unroll
      for (int r = 0; r < ROWS; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + c * dpad + g * ROWS + r);
        kc[r] = k4.x; kc[r + 1] = k4.y; kc[r + 2] = k4.z; kc[r + 3] = k4.w;
        if (!STATE_ONLY) {
          const float4 q4 = *reinterpret_cast<const float4*>(q_s + c * dpad + g * ROWS + r);
          qc[r] = q4.x; qc[r + 1] = q4.y; qc[r + 2] = q4.z; qc[r + 3] = q4.w;
        }
        if (FORM != FORM_SCALAR) {
          const float4 a4 = *reinterpret_cast<const float4*>(a_s + c * dpad + g * ROWS + r);
          ac[r] = a4.x; ac[r + 1] = a4.y; ac[r + 2] = a4.z; ac[r + 3] = a4.w;
        } else {
          ac[r] = ac[r + 1] = ac[r + 2] = ac[r + 3] = a_tok;
        }
      }
      if (STATE_ONLY) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) A[r] *= ac[r];
      }
      float o[COLS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
#pragma unroll
        for (int cc = 0; cc < COLS; ++cc) {
          const float kv = kc[r] * vv[cc];
          if (STATE_ONLY) {
            S[r][cc] = fmaf(ac[r], S[r][cc], kv);
          } else if (FORM == FORM_BONUS) {
            o[cc] = fmaf(fmaf(U[r], kv, S[r][cc]), qc[r], o[cc]);      // the old state plus the bonus for the current token
            S[r][cc] = fmaf(ac[r], S[r][cc], kv);
          } else {
            S[r][cc] = fmaf(ac[r], S[r][cc], kv);
            o[cc] = fmaf(S[r][cc], qc[r], o[cc]);
          }
        }
      }
      if (!STATE_ONLY) *reinterpret_cast<float4*>(part + (c * groups + g) * VT + j * COLS) = make_float4(o[0], o[1], o[2], o[3]);
    }
    if (STATE_ONLY) continue;                 // the first pass writes no outputs
    __syncthreads();
    for (int idx = tid; idx < n * VT; idx += nthreads) {
      const int c = idx / VT, jj = idx % VT, cc = blockIdx.x * VT + jj;
      if (cc >= vdim) continue;
      float o = 0.f;
      for (int gg = 0; gg < groups; ++gg) o += part[(c * groups + gg) * VT + jj];
      if (FORM == FORM_SCALAR) o = fmaf(skip, v_s[idx], o);
      a.out[(size_t)(c0 + c) * a.out_stride + (size_t)head * vdim + cc] = o;
    }
  }
  if (mode == 2 && !last) return;             // pass 2: only an entry's last segment ends at the request's new state
  float* S_out = mode == 1 ? S_seg : S_slot;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = g * ROWS + r;
    if (d >= dim) continue;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (col0 + c < vdim) S_out[(size_t)d * vdim + col0 + c] = S[r][c];
    if (mode == 1 && blockIdx.x == 0 && j == 0) a.seg_decay[(seg_index * a.heads + head) * dim + d] = A[r];
  }
}

// Chains the segments of every entry: seg_state[s] holds the segment's end state from zero on entry (but for an entry's
// last segment, which holds nothing) and its true start state on exit.  A thread per element of the state.
__global__ void __launch_bounds__(256)
scan_chain_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay, const float* __restrict__ state,
                  long long slot_stride, const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, int heads,
                  int dim, int vdim, int seg_len) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t per = (size_t)heads * dim * vdim;
  const size_t el = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (el >= per) return;
  const int entry = blockIdx.y;
  const size_t row = el / vdim;               // head * dim + d
  size_t seg0 = 0;
  for (int e = 0; e < entry; ++e) seg0 += (cu_tokens[e + 1] - cu_tokens[e] + seg_len - 1) / seg_len;
  const int n_seg = (cu_tokens[entry + 1] - cu_tokens[entry] + seg_len - 1) / seg_len;
  float S = state[(size_t)state_slots[entry] * slot_stride + el];
  // eight segments' loads are issued together; the chain itself is one multiply-add a segment
  for (int s0 = 0; s0 < n_seg; s0 += 8) {
    float local[8], decay[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool inner = s0 + i + 1 < n_seg;
      local[i] = inner ? seg_state[(seg0 + s0 + i) * per + el] : 0.f;
      decay[i] = inner ? seg_decay[(seg0 + s0 + i) * heads * dim + row] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (s0 + i >= n_seg) break;
      seg_state[(seg0 + s0 + i) * per + el] = S;
      S = fmaf(decay[i], S, local[i]);
    }
  }
}

#define SCAN_CHECK(name)                                                   \
  do {                                                                     \
    cudaError_t e__ = cudaPeekAtLastError();                               \
    if (e__ != cudaSuccess) {                                              \
      cudaGetLastError();                                                  \
      return llmk_fail((int)e__, "%s: %s", name, cudaGetErrorString(e__)); \
    }                                                                      \
  } while (0)

// seg_len > 0: two passes over segments with the chain between them; n_tokens is then the step's number of tokens and
// seg_state / seg_decay hold n_tokens / seg_len + n_entries segments.
template <typename T, int FORM>
int launch_scan(ScanArgs a, int n_entries, int n_tokens, int seg_len, float* seg_state, float* seg_decay, cudaStream_t stream) {
  constexpr int VT = 32;
  LLMK_REQUIRE(seg_len >= 0 && (seg_len == 0 || (seg_state && seg_decay && n_tokens > 0)), "scan: segments need their scratch");
  const int groups = (a.dim + ROWS - 1) / ROWS;
  const size_t smem = ((size_t)3 * CHUNK * groups * ROWS + CHUNK * VT + (size_t)CHUNK * groups * VT) * sizeof(float);
  if (smem > 48 * 1024)
  {
    cudaFuncSetAttribute(diag_scan_kernel<T, VT, FORM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(diag_scan_kernel<T, VT, FORM, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const int max_segs = seg_len ? (n_tokens - (n_entries - 1) + seg_len - 1) / seg_len : 1;
  LLMK_REQUIRE((long long)n_entries * max_segs <= 65535, "scan: too many segments for one launch");
  a.seg_len = seg_len; a.max_segs = max_segs; a.seg_state = seg_state; a.seg_decay = seg_decay;
  const dim3 grid((a.vdim + VT - 1) / VT, a.heads, n_entries * max_segs), block(VT / COLS, groups);
  for (int mode = seg_len ? 1 : 0; mode <= (seg_len ? 2 : 0); ++mode) {
    a.mode = mode;
    if (mode == 1)
      launch_kernel(diag_scan_kernel<T, VT, FORM, true>, grid, block, smem, stream, a);
    else
      launch_kernel(diag_scan_kernel<T, VT, FORM, false>, grid, block, smem, stream, a);
    SCAN_CHECK("diag_scan");
    if (mode == 1) {
      const size_t per = (size_t)a.heads * a.dim * a.vdim;
      launch_kernel(scan_chain_kernel, dim3((unsigned)((per + 255) / 256), n_entries), dim3(256), 0, stream, seg_state,
                    (const float*)seg_decay, (const float*)a.state, a.slot_stride, a.state_slots, a.cu_tokens, a.heads, a.dim,
                    a.vdim, seg_len);
      SCAN_CHECK("scan_chain");
    }
  }
  return 0;
}

// ---- token shift -------------------------------------------------------------------------------------------
// out[t, m, :] = h_t + (h_(t-1) - h_t) * mu[m, :] for m < mixes, h_(-1) of a request's first token being zero and
// that of a later step's first token the row kept in the state slot.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ h, long long h_stride,
                   const float* __restrict__ mu, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ state_slots, const int* __restrict__ token_entry, const int* __restrict__ cu_tokens,
                   int width, int mixes) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int e = token_entry[t];
  const bool first = t == cu_tokens[e];
  const float* st = state + (size_t)state_slots[e] * slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    const float cur = to_f32(h[(size_t)t * h_stride + c]);
    const float prev = first ? st[c] : to_f32(h[(size_t)(t - 1) * h_stride + c]);
    for (int m = 0; m < mixes; ++m)
      out[(size_t)t * out_stride + (size_t)m * width + c] = from_f32<T>(fmaf(prev - cur, mu[(size_t)m * width + c], cur));
  }
}

// ---- gated RMS norm over groups of channels ----------------------------------------------------------------
// out[t, g, :] = rms(x') * w[g, :] * gate' with x' = x (gate' = silu(gate)) or, gate_first, x' = x * silu(gate) (gate' = 1);
// x float32 [T, groups * n]; w [groups * n]; a warp per (t, g).
template <typename T>
__global__ void __launch_bounds__(128)
group_rmsnorm_gate_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, const T* __restrict__ gate,
                          long long gate_stride, long long items, int groups, int n, float eps, int gate_first) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / groups;
  const int g = (int)(item % groups);
  const float* row = x + (size_t)item * n;
  const T* gt = gate + (size_t)t * gate_stride + (size_t)g * n;
  float ss = 0.f;
  for (int c = lane; c < n; c += 32) {
    float v = row[c];
    if (gate_first) { const float z = to_f32(gt[c]); v *= z / (1.f + expf(-z)); }
    ss = fmaf(v, v, ss);
  }
  const float rstd = 1.f / sqrtf(warp_sum(ss) / (float)n + eps);
  for (int c = lane; c < n; c += 32) {
    const float z = to_f32(gt[c]);
    const float s = z / (1.f + expf(-z));
    out[(size_t)item * n + c] = from_f32<T>(row[c] * s * rstd * w[(size_t)g * n + c]);
  }
}

// ---- two mixers side by side -------------------------------------------------------------------------------
// out[t] = (rms(a[t]) * wa + rms(b[t]) * wb) / 2; a and b tensors or split-K partial results.  One CTA per token.
template <typename T>
__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(T* __restrict__ out, MaybePartial<T> a, MaybePartial<T> b, const float* __restrict__ wa,
                      const float* __restrict__ wb, int width, float eps) {
  extern __shared__ float rows_s[];            // [2][width]
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float va = a.at(base + c), vb = b.at(base + c);
    rows_s[c] = va; rows_s[width + c] = vb;
    sa = fmaf(va, va, sa); sb = fmaf(vb, vb, sb);
  }
  const float ra = 1.f / sqrtf(block_sum(sa, red) / (float)width + eps);
  const float rb = 1.f / sqrtf(block_sum(sb, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[base + c] = from_f32<T>(0.5f * (rows_s[c] * ra * wa[c] + rows_s[width + c] * rb * wb[c]));
}

}  // namespace

LLMK_API int llmk_token_shift(void* out, long long out_stride, const void* h, long long h_stride, const float* mu,
                              const float* state, long long slot_stride, const int* state_slots, const int* token_entry,
                              const int* cu_tokens, int n_tokens, int width, int mixes, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    const unsigned by = (unsigned)min(8, (width + 255) / 256);
    launch_kernel(token_shift_kernel<T>, dim3(n_tokens, by), dim3(256), 0, stream, (T*)out, out_stride, (const T*)h, h_stride,
                  mu, state, slot_stride, state_slots, token_entry, cu_tokens, width, mixes);
    LLMK_LAUNCH_CHECK("token_shift");
  });
}

// The bonus form.  r, k, v: column ranges of one projection result (row stride rkv_stride); z float32; shift_*: the input
// rows whose last one per entry is kept (float32 [shift_width] per slot) for the next step's token shift, or null.
LLMK_API int llmk_wkv_scan(float* out, long long out_stride, const void* r, const void* k, const void* v, long long rkv_stride,
                           const float* z, long long z_stride, const float* z_bias, const float* bonus, float* state,
                           long long slot_stride, const int* state_slots, const int* cu_tokens, int n_entries, int heads, int dim,
                           const void* shift_src, long long shift_stride, float* shift_state, long long shift_slot_stride,
                           int shift_width, int dtype, cudaStream_t stream, int n_tokens, int seg_len, float* seg_state,
                           float* seg_decay) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(dim > 0 && dim <= ROWS * MAX_GROUPS, "wkv_scan: head size %d (1 to %d)", dim, ROWS * MAX_GROUPS);
  ScanArgs a = {};
  a.out = out; a.out_stride = out_stride; a.q = r; a.k = k; a.v = v; a.qk_stride = a.v_stride = rkv_stride;
  a.z = z; a.z_stride = z_stride; a.z_bias = z_bias; a.bonus = bonus; a.state = state; a.slot_stride = slot_stride;
  a.state_slots = state_slots; a.cu_tokens = cu_tokens; a.heads = a.qk_heads = heads; a.dim = a.vdim = dim;
  a.shift_src = shift_src; a.shift_stride = shift_stride; a.shift_state = shift_state; a.shift_slot_stride = shift_slot_stride;
  a.shift_width = shift_width;
  return dispatch_dtype(dtype, [&](auto* tag) {
    return launch_scan<LLMK_ELEM(tag), FORM_BONUS>(a, n_entries, n_tokens, seg_len, seg_state, seg_decay, stream);
  });
}

// The scalar form.  x [T, heads * vdim], b and c [T, groups * dim] (one row stride bc_stride), dt [T, heads].
LLMK_API int llmk_ssd_scan(float* out, long long out_stride, const void* x, long long x_stride, const void* b, const void* c,
                           long long bc_stride, const void* dt, long long dt_stride, const float* dt_bias, const float* a_log,
                           const float* skip, float* state, long long slot_stride, const int* state_slots, const int* cu_tokens,
                           int n_entries, int heads, int groups, int dim, int vdim, int dtype, cudaStream_t stream, int n_tokens,
                           int seg_len, float* seg_state, float* seg_decay) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(dim > 0 && dim <= ROWS * MAX_GROUPS, "ssd_scan: state size %d (1 to %d)", dim, ROWS * MAX_GROUPS);
  LLMK_REQUIRE(groups > 0 && heads % groups == 0, "ssd_scan: %d heads do not divide into %d groups", heads, groups);
  ScanArgs a = {};
  a.out = out; a.out_stride = out_stride; a.q = c; a.k = b; a.v = x; a.qk_stride = bc_stride; a.v_stride = x_stride;
  a.dt = dt; a.dt_stride = dt_stride; a.dt_bias = dt_bias; a.a_log = a_log; a.skip = skip; a.state = state;
  a.slot_stride = slot_stride; a.state_slots = state_slots; a.cu_tokens = cu_tokens; a.heads = heads; a.qk_heads = groups;
  a.dim = dim; a.vdim = vdim;
  return dispatch_dtype(dtype, [&](auto* tag) {
    return launch_scan<LLMK_ELEM(tag), FORM_SCALAR>(a, n_entries, n_tokens, seg_len, seg_state, seg_decay, stream);
  });
}

// The gate form.  q [T, heads * dim] (silu is taken here) and v [T, heads * vdim] in the projections' kind with row strides of
// their own; z float32 [T, heads * dim] the forget gate's pre-activation, z_bias and lower float32 [heads * dim].
LLMK_API int llmk_gate_scan(float* out, long long out_stride, const void* q, long long q_stride, const void* v, long long v_stride,
                            const float* z, long long z_stride, const float* z_bias, const float* lower, float* state,
                            long long slot_stride, const int* state_slots, const int* cu_tokens, int n_entries, int heads, int dim,
                            int vdim, int dtype, cudaStream_t stream, int n_tokens, int seg_len, float* seg_state,
                            float* seg_decay) {
  if (n_entries == 0) return 0;
  LLMK_REQUIRE(dim > 0 && dim <= ROWS * MAX_GROUPS, "gate_scan: key size %d (1 to %d)", dim, ROWS * MAX_GROUPS);
  LLMK_REQUIRE(lower != nullptr && z != nullptr, "gate_scan: the gate's pre-activation and its lower bound are needed");
  ScanArgs a = {};
  a.out = out; a.out_stride = out_stride; a.q = q; a.k = nullptr; a.v = v; a.qk_stride = q_stride; a.v_stride = v_stride;
  a.z = z; a.z_stride = z_stride; a.z_bias = z_bias; a.bonus = lower; a.state = state; a.slot_stride = slot_stride;
  a.state_slots = state_slots; a.cu_tokens = cu_tokens; a.heads = a.qk_heads = heads; a.dim = dim; a.vdim = vdim;
  return dispatch_dtype(dtype, [&](auto* tag) {
    return launch_scan<LLMK_ELEM(tag), FORM_GATE>(a, n_entries, n_tokens, seg_len, seg_state, seg_decay, stream);
  });
}

LLMK_API int llmk_group_rmsnorm_gate(void* out, const float* x, const float* w, const void* gate, long long gate_stride,
                                     int n_tokens, int groups, int n, float eps, int gate_first, int dtype, cudaStream_t stream) {
  const long long items = (long long)n_tokens * groups;
  if (items == 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(group_rmsnorm_gate_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (T*)out, x, w,
                  (const T*)gate, gate_stride, items, groups, n, eps, gate_first);
    LLMK_LAUNCH_CHECK("group_rmsnorm_gate");
  });
}

LLMK_API int llmk_pair_norm_mean(void* out, const void* a, const float* a_parts, int a_splits, long long a_split_stride,
                                 const void* b, const float* b_parts, int b_splits, long long b_split_stride, const float* wa,
                                 const float* wb, int n_tokens, int width, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(width > 0 && width <= 12288, "pair_norm_mean: width %d (1 to 12288)", width);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    MaybePartial<T> ma{(const T*)a, a_parts, a_splits, a_split_stride}, mb{(const T*)b, b_parts, b_splits, b_split_stride};
    const size_t smem = (size_t)2 * width * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(pair_norm_mean_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(pair_norm_mean_kernel<T>, dim3(n_tokens), dim3(256), smem, stream, (T*)out, ma, mb, wa, wb, width, eps);
    LLMK_LAUNCH_CHECK("pair_norm_mean");
  });
}
