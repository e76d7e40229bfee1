// Kernels of mixers that carry a matrix of state per head and request:
//
//   shift mix          out[m][t] = x[t] + (x[t-1] - x[t]) * mu[m] for several mu at once;
//                      the row before a sequence's first token of the step comes from
//                      per-request state, which then takes the sequence's last row
//   low-rank decay     z[t][c] = b[c] + sum_r act(x[t][r]) * w2t[r][c], then
//                        form 0:  exp(-exp(z)),            act = tanh
//                        form 1:  sigmoid(z)^(1/tau),       act = identity
//                        form 2:  exp(-exp(A[c / per_head]) * softplus(z)), act = identity
//   linear recurrence  per (sequence, head), tokens in order, S [K][V] in fp32:
//                        plain form:  S = diag(w_t) S + k_t v_t^T;  o_t = S^T q_t
//                        bonus form:  o_t = (S + diag(u) k_t v_t^T)^T q_t;
//                                     S = diag(w_t) S + k_t v_t^T
//   head norm + gate   out[t][h] = o[t][h] / rms(o[t][h]) * gain * silu(gate[t][h])
//
// Everything is computed in fp32 with the accurate library functions; inputs that are
// projections arrive in the run's element type.
#include "common.cuh"
#include "elementwise_vec.cuh"

// ---------------------------------------------------------------------------
// shift mix.  One block per token.  The block of a sequence's first token reads the
// state row and afterwards stores the sequence's last row of this step there; each
// thread touches the same elements in both, so the read precedes the write.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void shift_mix_kernel(const TA* __restrict__ x, const float* __restrict__ mu,
                                 float* __restrict__ state, const int* __restrict__ cu_q,
                                 const int* __restrict__ seq_of_token,
                                 const int* __restrict__ state_slot, TA* __restrict__ out, int T,
                                 int W, int n_mix) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const bool first = (t == cu_q[s]);
  const TA* cur = x + (size_t)t * W;
  float* st = state + (size_t)state_slot[s] * W;
  const TA* last = x + (size_t)(cu_q[s + 1] - 1) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = to_f32(cur[i]);
    const float p = first ? st[i] : to_f32(cur[i - W]);
    const float d = p - v;
    for (int m = 0; m < n_mix; ++m)
      out[((size_t)m * T + t) * W + i] = from_f32<TA>(v + d * mu[(size_t)m * W + i]);
    if (first) st[i] = to_f32(last[i]);
  }
}

// bf16, width a multiple of 8: eight values a thread, 16-byte accesses
__global__ void shift_mix_bf16_vec_kernel(const uint4* __restrict__ x, const float* __restrict__ mu,
                                          float* __restrict__ state, const int* __restrict__ cu_q,
                                          const int* __restrict__ seq_of_token,
                                          const int* __restrict__ state_slot,
                                          uint4* __restrict__ out, int T, int W, int n_mix) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const bool first = (t == cu_q[s]);
  const int chunks = W >> 3;
  const uint4* cur = x + (size_t)t * chunks;
  float4* st = reinterpret_cast<float4*>(state + (size_t)state_slot[s] * W);
  const uint4* last = x + (size_t)(cu_q[s + 1] - 1) * chunks;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float v[8], p[8], f[8];
    bf8_to_f32(cur[c], v);
    if (first) {
      const float4 a = st[2 * c], b = st[2 * c + 1];
      p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
      p[4] = b.x; p[5] = b.y; p[6] = b.z; p[7] = b.w;
    } else {
      bf8_to_f32(cur[c - chunks], p);
    }
    for (int m = 0; m < n_mix; ++m) {
      const float4* mm = reinterpret_cast<const float4*>(mu + (size_t)m * W);
      const float4 a = mm[2 * c], b = mm[2 * c + 1];
      const float g[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = v[j] + (p[j] - v[j]) * g[j];
      out[((size_t)m * T + t) * chunks + c] = f32_to_bf8(f);
    }
    if (first) {
      bf8_to_f32(last[c], f);
      st[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
      st[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
}

IX_API int ix_shift_mix(const void* x, int dtype, const float* mu, float* state, const int* cu_q,
                        const int* seq_of_token, const int* state_slot, void* out, int T, int W,
                        int n_mix, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0 || n_mix <= 0) return IX_ERR_SIZE;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == IX_BF16 && W % 8 == 0 &&
      (((uintptr_t)x | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
    ix_launch(shift_mix_bf16_vec_kernel, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream,
              (const uint4*)x, mu, state, cu_q, seq_of_token, state_slot, (uint4*)out, T, W, n_mix);
    return ix_launch_status();
  }
  IX_DISPATCH_DTYPE(dtype, TA,
                    ix_launch(shift_mix_kernel<TA>, dim3(T), dim3(threads), 0, stream,
                              (const TA*)x, mu, state, cu_q, seq_of_token, state_slot, (TA*)out,
                              T, W, n_mix));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// low-rank decay.  A block takes LRD_TOKENS tokens and LRD_THREADS channels; a thread
// reads its channel's column of the transposed matrix w2t [R][C] once for all of the
// block's tokens (neighbouring threads read neighbouring addresses).  A token's sum runs
// over r in ascending order whatever else is in the block.
// ---------------------------------------------------------------------------
#define LRD_TOKENS 16
#define LRD_THREADS 128

template <typename TX>
__global__ void lowrank_decay_kernel(const TX* __restrict__ x, long long ldx,
                                     const float* __restrict__ w2t, const float* __restrict__ b,
                                     float* __restrict__ out, int T, int C, int R, int form,
                                     float inv_tau, const float* __restrict__ head_param,
                                     int per_head) {
  extern __shared__ __align__(16) float act[];   // [LRD_TOKENS][R]
  IX_PDL_WAIT();
  const int t0 = blockIdx.x * LRD_TOKENS;
  const int nt = min(LRD_TOKENS, T - t0);
  for (int i = threadIdx.x; i < nt * R; i += blockDim.x) {
    const float v = to_f32(x[(size_t)(t0 + i / R) * ldx + i % R]);
    act[i] = form == 0 ? tanhf(v) : v;
  }
  __syncthreads();
  const int c = blockIdx.y * LRD_THREADS + threadIdx.x;
  if (c >= C) return;
  float z[LRD_TOKENS];
#pragma unroll
  for (int j = 0; j < LRD_TOKENS; ++j) z[j] = 0.f;
  if ((R & 3) == 0) {       // four inner entries a shared-memory read; the same order of sums
    for (int r = 0; r < R; r += 4) {
      const float w0 = w2t[(size_t)r * C + c], w1 = w2t[(size_t)(r + 1) * C + c];
      const float w2 = w2t[(size_t)(r + 2) * C + c], w3 = w2t[(size_t)(r + 3) * C + c];
#pragma unroll
      for (int j = 0; j < LRD_TOKENS; ++j) {
        if (j < nt) {
          const float4 a = *reinterpret_cast<const float4*>(act + j * R + r);
          z[j] += a.x * w0;
          z[j] += a.y * w1;
          z[j] += a.z * w2;
          z[j] += a.w * w3;
        }
      }
    }
  } else {
    for (int r = 0; r < R; ++r) {
      const float w = w2t[(size_t)r * C + c];
#pragma unroll
      for (int j = 0; j < LRD_TOKENS; ++j)
        if (j < nt) z[j] += act[j * R + r] * w;
    }
  }
  const float bias = b ? b[c] : 0.f;
  const float neg_rate = form == 2 ? -expf(head_param[c / per_head]) : 0.f;
#pragma unroll
  for (int j = 0; j < LRD_TOKENS; ++j) {
    if (j >= nt) break;
    const float v = z[j] + bias;
    float d;
    if (form == 0) {
      d = expf(-expf(v));
    } else if (form == 2) {
      d = expf(neg_rate * (v > 20.f ? v : log1pf(expf(v))));
    } else {
      // log sigmoid(v) = min(v, 0) - log(1 + exp(-|v|))
      d = expf((fminf(v, 0.f) - log1pf(expf(-fabsf(v)))) * inv_tau);
    }
    out[(size_t)(t0 + j) * C + c] = d;
  }
}

IX_API int ix_lowrank_decay(const void* x, int x_dtype, long long ldx, const float* w2t,
                            const float* b, float* out, int T, int C, int R, int form, float tau,
                            const float* head_param, int per_head, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (C <= 0 || R <= 0 || ldx < R || form < 0 || form > 2 || !(tau > 0.f)) return IX_ERR_SIZE;
  if (form == 2 && (!head_param || per_head <= 0 || C % per_head)) return IX_ERR_SIZE;
  const size_t smem = (size_t)LRD_TOKENS * R * sizeof(float);
  if (smem > 48 * 1024) return IX_ERR_SMEM;
  dim3 grid((T + LRD_TOKENS - 1) / LRD_TOKENS, (C + LRD_THREADS - 1) / LRD_THREADS);
  if (grid.y > 65535) return IX_ERR_SIZE;
  IX_DISPATCH_DTYPE(x_dtype, TX,
                    ix_launch(lowrank_decay_kernel<TX>, grid, dim3(LRD_THREADS), smem, stream,
                              (const TX*)x, ldx, w2t, b, out, T, C, R, form, 1.0f / tau,
                              head_param, per_head));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// linear recurrence.  grid (ceil(V / 32) * segments, heads, sequences); a block is 32
// value columns times KS slices of the key channels (one warp per slice).  A thread keeps
// its KPT entries of one state column in registers while it walks its tokens; key channels
// do not interact, so the slices walk a chunk of tokens without meeting, leave their
// partial outputs in shared memory, and the partials are added in ascending slice order.
//
// Three forms of the walk:
//   whole (segments = 1)  a block walks all of its sequence's tokens of the step, from the
//                         state in the slot to the state it leaves there.  The order of
//                         every sum is fixed by (K, KS): a position's output does not
//                         depend on how its sequence was cut into steps or chunks.
//   local                 long prompts are cut into segments of seg_len tokens that are
//                         walked side by side.  The first pass walks every segment but a
//                         sequence's last from a zero state and leaves in scratch the
//                         state it ends with and the product of its decays (entry seg + 1);
//                         entry 0 takes the state from the slot.
//   joined                the second pass rebuilds a segment's start state from the
//                         entries before it, S <- P_i S + S_i in ascending i, then walks
//                         the segment with outputs; the last segment leaves the state.
// ---------------------------------------------------------------------------
#define LR_COLS 32
#define LR_CHUNK 16
#define LR_PF 4
enum { LR_WHOLE = 0, LR_LOCAL = 1, LR_JOINED = 2 };

// One state entry, one token.  The roundings are spelled out (one product, two fused
// multiply-adds; three in the bonus form), so that every path through the kernel - staged
// chunks, vector reads, the single-token form, the pass without outputs - rounds alike.
template <bool BONUS>
__device__ __forceinline__ void lr_step(float& S, float u, float kk, float w, float q, float vj,
                                        float& acc) {
  const float kv = __fmul_rn(kk, vj);
  if (BONUS) {
    acc = __fmaf_rn(__fmaf_rn(u, kv, S), q, acc);
    S = __fmaf_rn(w, S, kv);
  } else {
    S = __fmaf_rn(w, S, kv);
    acc = __fmaf_rn(S, q, acc);
  }
}
__device__ __forceinline__ void lr_step_local(float& S, float kk, float w, float vj) {
  S = __fmaf_rn(w, S, __fmul_rn(kk, vj));
}

template <typename TA, int KPT, bool BONUS, int MODE>
__global__ void __launch_bounds__(LR_COLS * 8, KPT <= 8 ? 4 : (KPT <= 16 ? 3 : 1))
linear_recurrence_kernel(const TA* __restrict__ q, long long ldq, const TA* __restrict__ k,
                         long long ldk, const TA* __restrict__ v, long long ldv,
                         const float* __restrict__ decay, const float* __restrict__ bonus,
                         float* __restrict__ state, const int* __restrict__ cu_q,
                         const int* __restrict__ state_slot, float* __restrict__ out, int H,
                         int K, int V, int KS, float q_scale, int seg_len, int nseg,
                         float* __restrict__ scr_s, float* __restrict__ scr_p) {
  constexpr int mode = MODE;
  extern __shared__ __align__(16) float sm[];
  float* q_s = sm;                       // [LR_CHUNK][K]
  float* k_s = q_s + LR_CHUNK * K;       // [LR_CHUNK][K]
  float* w_s = k_s + LR_CHUNK * K;       // [LR_CHUNK][K]
  float* v_s = w_s + LR_CHUNK * K;       // [LR_CHUNK][LR_COLS]
  float* part = v_s + LR_CHUNK * LR_COLS;  // [KS][LR_CHUNK][LR_COLS]
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31, ks = threadIdx.x >> 5;
  const int vtiles = (V + LR_COLS - 1) / LR_COLS;
  const int seg = blockIdx.x / vtiles;
  const int v0 = (blockIdx.x % vtiles) * LR_COLS, h = blockIdx.y, s = blockIdx.z;
  const int col = v0 + lane;
  const bool col_ok = col < V;
  const int seq_begin = cu_q[s], seq_end = cu_q[s + 1];
  const int nseg_s = mode == LR_WHOLE ? 1 : (seq_end - seq_begin + seg_len - 1) / seg_len;
  if (seg >= nseg_s) return;
  const int t_begin = mode == LR_WHOLE ? seq_begin : seq_begin + seg * seg_len;
  const int t_end = mode == LR_WHOLE ? seq_end : min(seq_end, t_begin + seg_len);
  float* st = state + ((size_t)state_slot[s] * H + h) * K * V;
  float* my_s = scr_s + ((size_t)s * H + h) * nseg * K * V;    // entries of this (sequence, head)
  float* my_p = scr_p + ((size_t)s * H + h) * nseg * K;
  const int kk0 = ks * KPT;
  const bool vec4 = (K & 3) == 0;      // then kk0 and every row of q_s, k_s, w_s are 16-byte marks
  const bool walks = mode != LR_LOCAL || seg < nseg_s - 1;

  float S[KPT], u[KPT], P[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    const bool ok = kk < K && col_ok;
    P[i] = 1.f;
    u[i] = (BONUS && kk < K) ? bonus[(size_t)h * K + kk] : 0.f;
    if (mode == LR_WHOLE) {
      S[i] = ok ? st[(size_t)kk * V + col] : 0.f;
    } else if (mode == LR_LOCAL) {
      if (seg == 0 && ok) my_s[(size_t)kk * V + col] = st[(size_t)kk * V + col];
      S[i] = 0.f;
    } else {
      S[i] = ok ? my_s[(size_t)kk * V + col] : 0.f;
    }
  }
  if (mode == LR_JOINED) {
    for (int e = 1; e <= seg; ++e) {
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const int kk = kk0 + i;
        if (kk < K && col_ok)
          S[i] = my_p[(size_t)e * K + kk] * S[i] + my_s[((size_t)e * K + kk) * V + col];
      }
    }
  }
  if (!walks) return;

  // A sequence that brings one token (a decode step): nothing is staged.  Every thread reads
  // its slice of q, k and the decay straight from global memory (the lanes of a warp read
  // the same addresses), the slices' partial outputs meet in shared memory once.  The same
  // operations in the same order as the walk below, so the same bits.
  if (mode == LR_WHOLE && t_end - t_begin == 1) {
    const size_t t = (size_t)t_begin;
    const float vj = col_ok ? to_f32(v[t * ldv + (size_t)h * V + col]) : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      const int kk = kk0 + i;
      if (kk < K) {
        const float qv = __fmul_rn(to_f32(q[t * ldq + (size_t)h * K + kk]), q_scale);
        lr_step<BONUS>(S[i], u[i], to_f32(k[t * ldk + (size_t)h * K + kk]),
                       decay[(t * H + h) * K + kk], qv, vj, acc);
      }
    }
    part[ks * LR_COLS + lane] = acc;
    __syncthreads();
    if (ks == 0 && col_ok) {
      float total = 0.f;
      for (int w = 0; w < KS; ++w) total += part[w * LR_COLS + lane];
      out[(t * H + h) * V + col] = total;
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      const int kk = kk0 + i;
      if (kk < K && col_ok) st[(size_t)kk * V + col] = S[i];
    }
    return;
  }

  // Where a chunk's inputs are at most LR_PF values a thread (key sizes up to 64 with eight
  // warps), the next chunk is fetched into registers while this one is walked, so that the
  // latency of global memory is not waited for at every chunk.
  const bool prefetch = LR_CHUNK * K <= LR_PF * (int)blockDim.x &&
                        LR_CHUNK * LR_COLS <= LR_PF * (int)blockDim.x;
  float pq[LR_PF], pk[LR_PF], pw[LR_PF], pv[LR_PF];
  auto fetch = [&](int t0, int n) {
#pragma unroll
    for (int e = 0; e < LR_PF; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < n * K) {
        const int c = i / K, kk = i % K;
        const size_t t = (size_t)(t0 + c);
        if (mode != LR_LOCAL) pq[e] = __fmul_rn(to_f32(q[t * ldq + (size_t)h * K + kk]), q_scale);
        pk[e] = to_f32(k[t * ldk + (size_t)h * K + kk]);
        pw[e] = decay[(t * H + h) * K + kk];
      }
      if (i < n * LR_COLS) {
        const int c = i / LR_COLS, j = i % LR_COLS;
        pv[e] = (v0 + j < V) ? to_f32(v[(size_t)(t0 + c) * ldv + (size_t)h * V + v0 + j]) : 0.f;
      }
    }
  };
  if (prefetch) fetch(t_begin, min(LR_CHUNK, t_end - t_begin));

  for (int t0 = t_begin; t0 < t_end; t0 += LR_CHUNK) {
    const int n = min(LR_CHUNK, t_end - t0);
    if (prefetch) {
#pragma unroll
      for (int e = 0; e < LR_PF; ++e) {
        const int i = threadIdx.x + e * blockDim.x;
        if (i < n * K) {
          if (mode != LR_LOCAL) q_s[i] = pq[e];
          k_s[i] = pk[e];
          w_s[i] = pw[e];
        }
        if (i < n * LR_COLS) v_s[i] = pv[e];
      }
    } else {
      for (int i = threadIdx.x; i < n * K; i += blockDim.x) {
        const int c = i / K, kk = i % K;
        const size_t t = (size_t)(t0 + c);
        if (mode != LR_LOCAL) q_s[i] = __fmul_rn(to_f32(q[t * ldq + (size_t)h * K + kk]), q_scale);
        k_s[i] = to_f32(k[t * ldk + (size_t)h * K + kk]);
        w_s[i] = decay[(t * H + h) * K + kk];
      }
      for (int i = threadIdx.x; i < n * LR_COLS; i += blockDim.x) {
        const int c = i / LR_COLS, j = i % LR_COLS;
        v_s[i] = (v0 + j < V) ? to_f32(v[(size_t)(t0 + c) * ldv + (size_t)h * V + v0 + j]) : 0.f;
      }
    }
    __syncthreads();
    if (prefetch && t0 + LR_CHUNK < t_end)
      fetch(t0 + LR_CHUNK, min(LR_CHUNK, t_end - t0 - LR_CHUNK));
    if (mode == LR_LOCAL) {
#pragma unroll 4
      for (int c = 0; c < n; ++c) {
        const float vj = v_s[c * LR_COLS + lane];
        const float* kc = k_s + c * K + kk0;
        const float* wc = w_s + c * K + kk0;
        if (vec4) {      // K a multiple of 4: four channels a shared-memory read
#pragma unroll
          for (int i = 0; i < KPT; i += 4) {
            if (kk0 + i < K) {
              const float4 k4 = *reinterpret_cast<const float4*>(kc + i);
              const float4 w4 = *reinterpret_cast<const float4*>(wc + i);
              lr_step_local(S[i], k4.x, w4.x, vj);
              lr_step_local(S[i + 1], k4.y, w4.y, vj);
              lr_step_local(S[i + 2], k4.z, w4.z, vj);
              lr_step_local(S[i + 3], k4.w, w4.w, vj);
              P[i] *= w4.x; P[i + 1] *= w4.y; P[i + 2] *= w4.z; P[i + 3] *= w4.w;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < KPT; ++i) {
            if (kk0 + i < K) {
              lr_step_local(S[i], kc[i], wc[i], vj);
              P[i] *= wc[i];
            }
          }
        }
      }
      __syncthreads();
      continue;
    }
#pragma unroll 4
    for (int c = 0; c < n; ++c) {
      const float vj = v_s[c * LR_COLS + lane];
      const float* qc = q_s + c * K + kk0;
      const float* kc = k_s + c * K + kk0;
      const float* wc = w_s + c * K + kk0;
      float acc = 0.f;
#define LR_STEP(SI, UI, KV, WV, QV) lr_step<BONUS>(SI, UI, KV, WV, QV, vj, acc);
      if (vec4) {        // K a multiple of 4: four channels a shared-memory read
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
          if (kk0 + i < K) {
            const float4 k4 = *reinterpret_cast<const float4*>(kc + i);
            const float4 w4 = *reinterpret_cast<const float4*>(wc + i);
            const float4 q4 = *reinterpret_cast<const float4*>(qc + i);
            LR_STEP(S[i], u[i], k4.x, w4.x, q4.x)
            LR_STEP(S[i + 1], u[i + 1], k4.y, w4.y, q4.y)
            LR_STEP(S[i + 2], u[i + 2], k4.z, w4.z, q4.z)
            LR_STEP(S[i + 3], u[i + 3], k4.w, w4.w, q4.w)
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < KPT; ++i) {
          if (kk0 + i < K) LR_STEP(S[i], u[i], kc[i], wc[i], qc[i])
        }
      }
#undef LR_STEP
      part[(ks * LR_CHUNK + c) * LR_COLS + lane] = acc;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * LR_COLS; i += blockDim.x) {
      const int c = i / LR_COLS, j = i % LR_COLS;
      if (v0 + j < V) {
        float total = 0.f;
        for (int w = 0; w < KS; ++w) total += part[(w * LR_CHUNK + c) * LR_COLS + j];
        out[((size_t)(t0 + c) * H + h) * V + v0 + j] = total;
      }
    }
    __syncthreads();
  }
  if (mode == LR_LOCAL) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      const int kk = kk0 + i;
      if (kk < K && col_ok) my_s[((size_t)(seg + 1) * K + kk) * V + col] = S[i];
      if (kk < K && v0 == 0 && lane == 0) my_p[(size_t)(seg + 1) * K + kk] = P[i];
    }
    return;
  }
  if (mode == LR_JOINED && seg != nseg_s - 1) return;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    if (kk < K && col_ok) st[(size_t)kk * V + col] = S[i];
  }
}

IX_API int ix_linear_recurrence_max_dim() { return 8 * 64; }

// Floats of scratch the segmented walk needs for `S` sequences cut into `nseg` segments.
IX_API long long ix_linear_recurrence_scratch_floats(int S, int H, int K, int V, int nseg) {
  return nseg <= 1 ? 0 : (long long)S * H * nseg * ((long long)K * V + K);
}

template <typename TA, int KPT>
static void launch_recurrence(const void* q, long long ldq, const void* k, long long ldk,
                              const void* v, long long ldv, const float* decay,
                              const float* bonus, float* state, const int* cu_q,
                              const int* state_slot, float* out, int S, int H, int K, int V,
                              int KS, float q_scale, int bonus_form, size_t smem, int seg_len,
                              int nseg, float* scratch, cudaStream_t stream) {
  const int vtiles = (V + LR_COLS - 1) / LR_COLS;
  dim3 grid(vtiles * nseg, H, S), block(LR_COLS * KS);
  float* scr_s = scratch;
  float* scr_p = scratch ? scratch + (size_t)S * H * nseg * K * V : nullptr;
  auto go = [&](auto kern, int seg_len_, int nseg_) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ix_launch(kern, grid, block, smem, stream, (const TA*)q, ldq, (const TA*)k, ldk, (const TA*)v,
              ldv, decay, bonus, state, cu_q, state_slot, out, H, K, V, KS, q_scale, seg_len_,
              nseg_, scr_s, scr_p);
  };
  if (nseg <= 1) {
    if (bonus_form) go(linear_recurrence_kernel<TA, KPT, true, LR_WHOLE>, 0, 1);
    else go(linear_recurrence_kernel<TA, KPT, false, LR_WHOLE>, 0, 1);
    return;
  }
  go(linear_recurrence_kernel<TA, KPT, false, LR_LOCAL>, seg_len, nseg);
  if (bonus_form) go(linear_recurrence_kernel<TA, KPT, true, LR_JOINED>, seg_len, nseg);
  else go(linear_recurrence_kernel<TA, KPT, false, LR_JOINED>, seg_len, nseg);
}

// seg_len, nseg: 0, 1 for the walk from end to end; otherwise every sequence is cut into
// segments of seg_len tokens (nseg covers the longest) and `scratch` holds
// ix_linear_recurrence_scratch_floats(...) floats.
IX_API int ix_linear_recurrence(const void* q, long long ldq, const void* k, long long ldk,
                                const void* v, long long ldv, int dtype, const float* decay,
                                const float* bonus, float* state, const int* cu_q,
                                const int* state_slot, float* out, int S, int H, int K, int V,
                                float q_scale, int bonus_form, int seg_len, int nseg,
                                float* scratch, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (H <= 0 || K <= 0 || V <= 0 || K > 8 * 64 || H > 65535 || S > 65535) return IX_ERR_SIZE;
  if (bonus_form && !bonus) return IX_ERR_SIZE;
  if (nseg < 1 || (nseg > 1 && (seg_len <= 0 || !scratch))) return IX_ERR_SIZE;
  const int KS = K > 32 ? 8 : (K > 8 ? 4 : 1);
  const int kpt = (K + KS - 1) / KS;
  const size_t smem =
      ((size_t)3 * LR_CHUNK * K + LR_CHUNK * LR_COLS + (size_t)KS * LR_CHUNK * LR_COLS) *
      sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
#define LR_GO(KPT)                                                                              \
  IX_DISPATCH_DTYPE(dtype, TA,                                                                  \
                    (launch_recurrence<TA, KPT>(q, ldq, k, ldk, v, ldv, decay, bonus, state,    \
                                                cu_q, state_slot, out, S, H, K, V, KS, q_scale, \
                                                bonus_form, smem, seg_len, nseg, scratch,       \
                                                stream)))
  if (kpt <= 8) LR_GO(8);
  else if (kpt <= 16) LR_GO(16);
  else if (kpt <= 32) LR_GO(32);
  else LR_GO(64);
#undef LR_GO
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// head norm + gate.  One warp per (token, head).  `gain` covers all heads
// (gain_per_head) or is shared by them.  gate_form 0: silu(gate); 1: sigmoid(gate).
// ---------------------------------------------------------------------------
#define HNG_WARPS 4

template <typename TG, typename TA>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain,
                                      int gain_per_head, const TG* __restrict__ gate,
                                      long long ldg, TA* __restrict__ out, int H, int V,
                                      float eps, int gate_form) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int h = blockIdx.y * HNG_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (h >= H) return;
  const float* row = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += row[c] * row[c];
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
  const float* g = gain + (gain_per_head ? (size_t)h * V : 0);
  const TG* gt = gate + (size_t)t * ldg + (size_t)h * V;
  TA* dst = out + ((size_t)t * H + h) * V;
  for (int c = lane; c < V; c += 32) {
    const float z = to_f32(gt[c]);
    const float sg = 1.0f / (1.0f + expf(-z));
    dst[c] = from_f32<TA>(row[c] * inv * g[c] * (gate_form ? sg : z * sg));
  }
}

// bf16 gate and output, V a multiple of 4 with V / 4 a power of two up to 32: GL = V / 4
// lanes share a head, each with four values (16-byte reads of o and the gain, 8-byte ones
// of the gate), 32 / GL heads a warp.  The sum of squares is added by a shuffle tree inside
// the lanes of a head.
template <int GL>
__global__ void head_norm_gate_bf16_vec_kernel(const float* __restrict__ o,
                                               const float* __restrict__ gain, int gain_per_head,
                                               const bf16* __restrict__ gate, long long ldg,
                                               bf16* __restrict__ out, int H, int V, float eps) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  constexpr int HPW = 32 / GL;
  const int h = (blockIdx.y * HNG_WARPS + (threadIdx.x >> 5)) * HPW + lane / GL;
  const int sub = lane % GL;
  const bool ok = h < H;
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
  if (ok) x = reinterpret_cast<const float4*>(o + ((size_t)t * H + h) * V)[sub];
  float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
#pragma unroll
  for (int d = GL / 2; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if (!ok) return;
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  const float4 g = reinterpret_cast<const float4*>(gain + (gain_per_head ? (size_t)h * V : 0))[sub];
  const uint2 zr = reinterpret_cast<const uint2*>(gate + (size_t)t * ldg + (size_t)h * V)[sub];
  const float2 z01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zr.x));
  const float2 z23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zr.y));
  const float r0 = x.x * inv * g.x * (z01.x / (1.0f + expf(-z01.x)));
  const float r1 = x.y * inv * g.y * (z01.y / (1.0f + expf(-z01.y)));
  const float r2 = x.z * inv * g.z * (z23.x / (1.0f + expf(-z23.x)));
  const float r3 = x.w * inv * g.w * (z23.y / (1.0f + expf(-z23.y)));
  uint2 w;
  *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(r0, r1);
  *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(r2, r3);
  reinterpret_cast<uint2*>(out + ((size_t)t * H + h) * V)[sub] = w;
}

IX_API int ix_head_norm_gate(const float* o, const float* gain, int gain_per_head,
                             const void* gate, int gate_dtype, long long ldg, void* out,
                             int out_dtype, int T, int H, int V, float eps, int gate_form,
                             cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || V <= 0 || ldg < (long long)H * V) return IX_ERR_SIZE;
  const int groups = (H + HNG_WARPS - 1) / HNG_WARPS;
  if (groups > 65535) return IX_ERR_SIZE;
  if (gate_dtype != out_dtype) return IX_ERR_UNSUPPORTED;
  const int gl = V / 4;
  if (gate_form == 0 && out_dtype == IX_BF16 && V % 4 == 0 && gl <= 32 && (gl & (gl - 1)) == 0 && ldg % 4 == 0 &&
      (((uintptr_t)o | (uintptr_t)gain) & 15) == 0 && (((uintptr_t)gate | (uintptr_t)out) & 7) == 0) {
    const int hpb = HNG_WARPS * (32 / gl);
    const int vgroups = (H + hpb - 1) / hpb;
#define IX_HNG(GL)                                                                            \
  ix_launch(head_norm_gate_bf16_vec_kernel<GL>, dim3(T, vgroups), dim3(32 * HNG_WARPS), 0,    \
            stream, o, gain, gain_per_head, (const bf16*)gate, ldg, (bf16*)out, H, V, eps)
    if (gl == 32) IX_HNG(32);
    else if (gl == 16) IX_HNG(16);
    else if (gl == 8) IX_HNG(8);
    else if (gl == 4) IX_HNG(4);
    else if (gl == 2) IX_HNG(2);
    else IX_HNG(1);
#undef IX_HNG
    return ix_launch_status();
  }
  IX_DISPATCH_DTYPE(out_dtype, TA,
                    ix_launch(head_norm_gate_kernel<TA, TA>, dim3(T, groups),
                              dim3(32 * HNG_WARPS), 0, stream, o, gain, gain_per_head,
                              (const TA*)gate, ldg, (TA*)out, H, V, eps, gate_form));
  return ix_launch_status();
}
