// Kernels of layers built around a short causal convolution and a recurrence with a
// matrix of state per head and request, and of the pre-norm arrangement with a scaled
// residual and a centred norm:
//
//   add + norm          resid += scale * delta (+ vector); out = norm(resid) * gain, where
//                       norm subtracts the mean (layer norm) or not (RMS norm)
//   stream concat       out[t] = [resid[t] + scale * delta[t] ; first[t]] in the run's type
//   causal convolution  y[t][c] = act(b[c] + sum_j w[c][j] x[t - (taps-1) + j][c]) with the
//                       taps-1 inputs before a sequence's first token of the step taken
//                       from per-request state, which a second kernel then moves on
//   state space         S = exp(-exp(A) dt) S + dt B x^T;  y = S^T C + D x   (scalar decay)
//   gated delta rule    S = diag(g) S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q
//   gate + group norm   out = groupnorm(y * silu(z)) * gain
//   normed pair mean    out = (l / rms(l) * gl + r / rms(r) * gr) / 2
//   relu squared, table routing, scaling of rows
//
// Everything but the stored activations is fp32 with the accurate library functions.
#include "common.cuh"

// ---------------------------------------------------------------------------
// add + norm.  One block per output row; the row is kept in shared memory between the
// passes (mean, then the mean of squared deviations, then the output).
// ---------------------------------------------------------------------------
// four neighbouring entries at once (the address is a multiple of four entries)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&a);
  u.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// The same passes with four entries per access, for rows of a multiple of four entries on
// 16-byte boundaries.  A thread's partial sums run over other entries than in the form
// below: the two differ by rounding, and one row size always takes the same form.
template <typename TD, typename TO>
__global__ void add_scaled_norm_vec_kernel(float* __restrict__ resid,
                                           const TD* __restrict__ delta, float scale,
                                           const float* __restrict__ vector,
                                           const float* __restrict__ gain,
                                           const int* __restrict__ rows, TO* __restrict__ out,
                                           int H, float eps, int center, int write_back) {
  extern __shared__ __align__(16) float row_s[];   // [H] + 32
  float* scratch = row_s + H;
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  float sum = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = ld4(x + i);
    if (delta) {
      const float4 d = ld4(delta + src * H + i);
      v.x += scale * d.x, v.y += scale * d.y, v.z += scale * d.z, v.w += scale * d.w;
    }
    if (vector) {
      const float4 a = ld4(vector + i);
      v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
    }
    st4(row_s + i, v);
    if (write_back) st4(x + i, v);
    sum += (v.x + v.y) + (v.z + v.w);
  }
  float mean = 0.f;
  if (center) mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {   // a thread's own entries
    const float4 v = ld4(row_s + i);
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    sq += (a * a + b * b) + (c * c + d * d);
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = ld4(row_s + i), g = ld4(gain + i);
    st4(out + (size_t)r * H + i, make_float4((v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y,
                                             (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w));
  }
}

template <typename TD, typename TO>
__global__ void add_scaled_norm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                       float scale, const float* __restrict__ vector,
                                       const float* __restrict__ gain,
                                       const int* __restrict__ rows, TO* __restrict__ out, int H,
                                       float eps, int center, int write_back) {
  extern __shared__ __align__(16) float row_s[];   // [H] + 32
  float* scratch = row_s + H;
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  float sum = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (delta) v += scale * to_f32(delta[src * H + i]);
    if (vector) v += vector[i];
    row_s[i] = v;
    if (write_back) x[i] = v;
    sum += v;
  }
  float mean = 0.f;
  if (center) mean = block_sum(sum, scratch) / (float)H;
  else __syncthreads();
  float sq = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row_s[i] - mean;
    sq += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)r * H + i] = from_f32<TO>((row_s[i] - mean) * inv * gain[i]);
}

IX_API int ix_add_scaled_norm(float* resid, const void* delta, int delta_dtype, float scale,
                              const float* vector, const float* gain, const int* rows, void* out,
                              int out_dtype, int R, int H, float eps, int center, int write_back,
                              cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (H <= 0) return IX_ERR_SIZE;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  const auto at16 = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; };
  const bool vec = H % 4 == 0 && at16(resid) && at16(delta) && at16(vector) && at16(gain) &&
                   at16(out);
  const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128))
                          : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define IX_ASN(TD, TO)                                                                       \
  do {                                                                                       \
    auto kern = vec ? add_scaled_norm_vec_kernel<TD, TO> : add_scaled_norm_kernel<TD, TO>;   \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    ix_launch(kern, dim3(R), dim3(threads), smem, stream, resid, (const TD*)delta, scale,    \
              vector, gain, rows, (TO*)out, H, eps, center, write_back);                     \
  } while (0)
  if (out_dtype == IX_F32) {
    if (delta_dtype == IX_F32) IX_ASN(float, float);
    else if (delta_dtype == IX_BF16) IX_ASN(bf16, float);
    else return IX_ERR_DTYPE;
  } else if (out_dtype == IX_BF16) {
    if (delta_dtype == IX_F32) IX_ASN(float, bf16);
    else if (delta_dtype == IX_BF16) IX_ASN(bf16, bf16);
    else return IX_ERR_DTYPE;
  } else {
    return IX_ERR_DTYPE;
  }
#undef IX_ASN
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// stream concat: out[t] = [resid[t] + scale * delta[t] (+ vector) ; first[t]].
// ---------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void stream_concat_kernel(const float* __restrict__ resid,
                                     const TD* __restrict__ delta, float scale,
                                     const float* __restrict__ vector,
                                     const float* __restrict__ first, TO* __restrict__ out, int T,
                                     int H) {
  IX_PDL_WAIT();
  const size_t n = (size_t)T * H;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / H, c = i - t * H;
    float v = resid[i];
    if (delta) v += scale * to_f32(delta[i]);
    if (vector) v += vector[c];
    out[t * 2 * H + c] = from_f32<TO>(v);
    out[t * 2 * H + H + c] = from_f32<TO>(first[i]);
  }
}

IX_API int ix_stream_concat(const float* resid, const void* delta, int delta_dtype, float scale,
                            const float* vector, const float* first, void* out, int out_dtype,
                            int T, int H, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0) return IX_ERR_SIZE;
  const size_t n = (size_t)T * H;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
#define IX_SC(TD, TO)                                                                      \
  ix_launch(stream_concat_kernel<TD, TO>, dim3(blocks), dim3(256), 0, stream, resid,      \
            (const TD*)delta, scale, vector, first, (TO*)out, T, H)
  if (out_dtype == IX_F32) {
    if (delta_dtype == IX_F32) IX_SC(float, float);
    else IX_SC(bf16, float);
  } else if (out_dtype == IX_BF16) {
    if (delta_dtype == IX_F32) IX_SC(float, bf16);
    else IX_SC(bf16, bf16);
  } else {
    return IX_ERR_DTYPE;
  }
#undef IX_SC
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// causal convolution over time per channel.  x [T, C] is a view with row pitch ldx;
// w [C, taps] (the last column multiplies the current token); state [slots, taps-1, C]
// holds a request's last taps-1 inputs (oldest first).  A thread owns one channel of one
// token; the sum runs from the oldest tap to the newest whatever the step's cut.
// ---------------------------------------------------------------------------
#define CONV_THREADS 128
#define CONV_MAX_TAPS 16

template <typename TA>
__global__ void causal_conv_kernel(const TA* __restrict__ x, long long ldx,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state,
                                   const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ state_slot, TA* __restrict__ out,
                                   int C, int taps, int act) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int s = seq_of_token[t];
  const int begin = cu_q[s];
  const float* st = state + (size_t)state_slot[s] * (taps - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = t - (taps - 1) + j;          // token index of this tap's input
    float v;
    if (src >= begin) {
      v = to_f32(x[(size_t)src * ldx + c]);
    } else {
      // begin - src inputs back from the step's first token: 1 is the newest kept one
      const int back = begin - src;               // 1 .. taps-1
      v = st[(size_t)(taps - 1 - back) * C + c];
    }
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  if (act) acc = acc / (1.0f + expf(-acc));
  out[(size_t)t * C + c] = from_f32<TA>(acc);
}

// The same sums for long steps: a thread owns two neighbouring channels of CONV_RUN tokens in
// a row and keeps the last TAPS - 1 inputs in registers, so that an input is read once.  The
// window is filled as above at the run's first token and wherever a sequence begins inside
// the run; the sum of a token runs over the same terms in the same order as above, so the
// two kernels give the same bits.
#define CONV_RUN 16
template <typename TA> struct ConvPair;
template <> struct ConvPair<float> { typedef float2 type; };
template <> struct ConvPair<bf16> { typedef __nv_bfloat162 type; };
__device__ __forceinline__ float2 pair_f32(float2 v) { return v; }
__device__ __forceinline__ float2 pair_f32(__nv_bfloat162 v) {
  return make_float2(__low2float(v), __high2float(v));
}

template <typename TA, int TAPS>
__global__ void __launch_bounds__(CONV_THREADS)
causal_conv_run_kernel(const TA* __restrict__ x, long long ldx, const float* __restrict__ w,
                       const float* __restrict__ bias, const float* __restrict__ state,
                       const int* __restrict__ cu_q, const int* __restrict__ seq_of_token,
                       const int* __restrict__ state_slot, TA* __restrict__ out, int T, int C,
                       int act) {
  IX_PDL_WAIT();
  const int t0 = blockIdx.x * CONV_RUN;
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * 2;
  if (c >= C) return;
  float wv[2][TAPS], win[2][TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) {
    wv[0][j] = w[(size_t)c * TAPS + j];
    wv[1][j] = w[(size_t)(c + 1) * TAPS + j];
  }
  const float b0 = bias ? bias[c] : 0.f, b1 = bias ? bias[c + 1] : 0.f;
  // the run's inputs are all on their way before the first is used
  typedef typename ConvPair<TA>::type P2;
  P2 raw[CONV_RUN];
#pragma unroll
  for (int i = 0; i < CONV_RUN; ++i)
    if (t0 + i < T) raw[i] = *reinterpret_cast<const P2*>(x + (size_t)(t0 + i) * ldx + c);
#pragma unroll
  for (int i = 0; i < CONV_RUN; ++i) {
    const int t = t0 + i;
    if (t >= T) break;
    const int s = seq_of_token[t];
    const int begin = cu_q[s];
    if (t == t0 || t == begin) {
      const float* st = state + (size_t)state_slot[s] * (TAPS - 1) * C;
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) {
        const int src = t - (TAPS - 1) + j;
        if (src >= begin) {
          win[0][j] = to_f32(x[(size_t)src * ldx + c]);
          win[1][j] = to_f32(x[(size_t)src * ldx + c + 1]);
        } else {
          const int back = begin - src;
          win[0][j] = st[(size_t)(TAPS - 1 - back) * C + c];
          win[1][j] = st[(size_t)(TAPS - 1 - back) * C + c + 1];
        }
      }
    }
    const float2 cur = pair_f32(raw[i]);
    const float cur0 = cur.x, cur1 = cur.y;
    float a0 = b0, a1 = b1;
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {
      a0 = fmaf(wv[0][j], win[0][j], a0);
      a1 = fmaf(wv[1][j], win[1][j], a1);
    }
    a0 = fmaf(wv[0][TAPS - 1], cur0, a0);
    a1 = fmaf(wv[1][TAPS - 1], cur1, a1);
#pragma unroll
    for (int j = 0; j + 1 < TAPS - 1; ++j) {
      win[0][j] = win[0][j + 1];
      win[1][j] = win[1][j + 1];
    }
    if (TAPS > 1) {
      win[0][TAPS - 2] = cur0;
      win[1][TAPS - 2] = cur1;
    }
    if (act) {
      a0 = a0 / (1.0f + expf(-a0));
      a1 = a1 / (1.0f + expf(-a1));
    }
    if (sizeof(TA) == 2) {
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * C + c) = __floats2bfloat162_rn(a0, a1);
    } else {
      *reinterpret_cast<float2*>(out + (size_t)t * C + c) = make_float2(a0, a1);
    }
  }
}

// Steps of this many tokens or more take the kernel that walks runs of tokens.
#define CONV_RUN_MIN_TOKENS 1024

// The state moves on: entry i becomes the input taps-1-i tokens before the sequence's
// next token.  A thread owns one channel of one sequence and walks i upwards; what it
// reads from the old state lies above what it has written.
template <typename TA>
__global__ void conv_state_update_kernel(const TA* __restrict__ x, long long ldx,
                                         float* __restrict__ state, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slot, int C, int taps) {
  IX_PDL_WAIT();
  const int s = blockIdx.x;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  const int begin = cu_q[s], n = cu_q[s + 1] - begin;
  if (n <= 0) return;
  float* st = state + (size_t)state_slot[s] * (taps - 1) * C;
  for (int i = 0; i < taps - 1; ++i) {
    const int src = n - (taps - 1) + i;           // index among this step's tokens
    const float v = src >= 0 ? to_f32(x[(size_t)(begin + src) * ldx + c])
                             : st[(size_t)(i + n) * C + c];
    st[(size_t)i * C + c] = v;
  }
}

IX_API int ix_causal_conv(const void* x, int dtype, long long ldx, const float* w,
                          const float* bias, float* state, const int* cu_q,
                          const int* seq_of_token, const int* state_slot, void* out, int T, int S,
                          int C, int taps, int act, cudaStream_t stream) {
  if (T <= 0 || S <= 0) return IX_OK;
  if (C <= 0 || taps < 1 || taps > CONV_MAX_TAPS || ldx < C) return IX_ERR_SIZE;
  const int cb = (C + CONV_THREADS - 1) / CONV_THREADS;
  if (cb > 65535) return IX_ERR_SIZE;
  const size_t two = dtype == IX_F32 ? 8 : 4;
  const bool run = T >= CONV_RUN_MIN_TOKENS && taps >= 2 && taps <= 4 && C % 2 == 0 &&
                   ldx % 2 == 0 && (uintptr_t)x % two == 0 && (uintptr_t)out % two == 0;
  const dim3 rgrid((T + CONV_RUN - 1) / CONV_RUN, (C / 2 + CONV_THREADS - 1) / CONV_THREADS);
#define CONV_GO(TAPS)                                                                        \
  ix_launch(causal_conv_run_kernel<TA, TAPS>, rgrid, dim3(CONV_THREADS), 0, stream,          \
            (const TA*)x, ldx, w, bias, (const float*)state, cu_q, seq_of_token, state_slot, \
            (TA*)out, T, C, act)
  IX_DISPATCH_DTYPE(dtype, TA, {
    if (run && taps == 2) CONV_GO(2);
    else if (run && taps == 3) CONV_GO(3);
    else if (run && taps == 4) CONV_GO(4);
    else
      ix_launch(causal_conv_kernel<TA>, dim3(T, cb), dim3(CONV_THREADS), 0, stream,
                (const TA*)x, ldx, w, bias, (const float*)state, cu_q, seq_of_token,
                state_slot, (TA*)out, C, taps, act);
    if (taps > 1)
      ix_launch(conv_state_update_kernel<TA>, dim3(S, cb), dim3(CONV_THREADS), 0, stream,
                (const TA*)x, ldx, state, cu_q, state_slot, C, taps);
  });
#undef CONV_GO
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// The two recurrences.  grid (ceil(V / 32), heads, sequences); a block is 32 value columns
// times KS slices of the key (state) channels, one warp a slice.  A thread keeps its KPT
// entries of one state column in registers while it walks the sequence's tokens of the
// step in chunks of RC_CHUNK staged in shared memory.  A token's arithmetic depends on the
// token and the state alone, and every sum has an order fixed by (K, KS): a position's
// output does not depend on how its sequence was cut into steps or on the batch.
// ---------------------------------------------------------------------------
#define RC_COLS 32
#define RC_CHUNK 16

__device__ __forceinline__ float softplus_f(float z) {
  return z > 20.f ? z : log1pf(expf(z));
}

// state space: q = C, k = dt * B, scalar decay a = exp(-exp(A) dt), skip D x.  Slices do
// not interact inside a token, so they meet once per chunk.
//
// Three forms of the walk, as in the linear recurrence with a decay per key channel:
//   whole    a block walks all of its sequence's tokens of the step, from the state in the
//            slot to the state it leaves there.
//   local    long prompts are cut into segments of seg_len tokens that are walked side by
//            side (grid.x = value tiles * segments).  The first pass walks every segment
//            but a sequence's last from a zero state, without outputs, and leaves in scratch
//            the state it ends with and the product of its decays (entry seg + 1); entry 0
//            takes the state from the slot.
//   joined   the second pass rebuilds a segment's start state from the entries before it,
//            S <- P_i S + S_i in ascending i, walks the segment with outputs, and the last
//            segment leaves the state.  Against the whole walk the results differ by
//            rounding only.
enum { RC_WHOLE = 0, RC_LOCAL = 1, RC_JOINED = 2 };

template <typename TA, int KPT, int MODE>
__global__ void __launch_bounds__(RC_COLS * 8)
ssd_recurrence_kernel(const TA* __restrict__ xbc, long long ld, const TA* __restrict__ dt_raw,
                      long long ld_dt, const float* __restrict__ dt_bias,
                      const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      float* __restrict__ state, const int* __restrict__ cu_q,
                      const int* __restrict__ state_slot, float* __restrict__ out, int H, int V,
                      int K, int G, int KS, int seg_len, int nseg, float* __restrict__ scr_s,
                      float* __restrict__ scr_p) {
  extern __shared__ __align__(16) float sm[];
  float* c_s = sm;                          // [RC_CHUNK][K]   C_t
  float* k_s = c_s + RC_CHUNK * K;          // [RC_CHUNK][K]   dt * B_t
  float* v_s = k_s + RC_CHUNK * K;          // [RC_CHUNK][RC_COLS]  x_t
  float* a_s = v_s + RC_CHUNK * RC_COLS;    // [RC_CHUNK]
  float* part = a_s + RC_CHUNK;             // [KS][RC_CHUNK][RC_COLS]
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31, ks = threadIdx.x >> 5;
  const int vtiles = (V + RC_COLS - 1) / RC_COLS;
  const int seg = blockIdx.x / vtiles;
  const int v0 = (blockIdx.x % vtiles) * RC_COLS, h = blockIdx.y, s = blockIdx.z;
  const int col = v0 + lane;
  const bool col_ok = col < V;
  const int g = h / (H / G);
  const int inner = H * V;
  const int seq_begin = cu_q[s], seq_end = cu_q[s + 1];
  if (seq_end <= seq_begin) return;
  const int nseg_s = MODE == RC_WHOLE ? 1 : (seq_end - seq_begin + seg_len - 1) / seg_len;
  if (seg >= nseg_s) return;
  const int t_begin = MODE == RC_WHOLE ? seq_begin : seq_begin + seg * seg_len;
  const int t_end = MODE == RC_WHOLE ? seq_end : min(seq_end, t_begin + seg_len);
  float* st = state + ((size_t)state_slot[s] * H + h) * K * V;
  float* my_s = scr_s + ((size_t)s * H + h) * nseg * K * V;   // entries of this (sequence, head)
  float* my_p = scr_p + ((size_t)s * H + h) * nseg;
  const bool walks = MODE != RC_LOCAL || seg < nseg_s - 1;
  const int kk0 = ks * KPT;
  const float neg_a = -expf(a_log[h]), bias = dt_bias[h], dsk = d_skip[h];
  float S[KPT];
  float P = 1.f;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    const bool ok = kk < K && col_ok;
    if (MODE == RC_WHOLE) {
      S[i] = ok ? st[(size_t)kk * V + col] : 0.f;
    } else if (MODE == RC_LOCAL) {
      if (seg == 0 && ok) my_s[(size_t)kk * V + col] = st[(size_t)kk * V + col];
      S[i] = 0.f;
    } else {
      S[i] = ok ? my_s[(size_t)kk * V + col] : 0.f;
    }
  }
  if (MODE == RC_JOINED) {
    for (int e = 1; e <= seg; ++e) {
      const float pe = my_p[e];
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const int kk = kk0 + i;
        if (kk < K && col_ok) S[i] = pe * S[i] + my_s[((size_t)e * K + kk) * V + col];
      }
    }
  }
  if (!walks) return;
  for (int t0 = t_begin; t0 < t_end; t0 += RC_CHUNK) {
    const int n = min(RC_CHUNK, t_end - t0);
    if (threadIdx.x < n) {
      const float dt = softplus_f(to_f32(dt_raw[(size_t)(t0 + threadIdx.x) * ld_dt + h]) + bias);
      a_s[threadIdx.x] = expf(neg_a * dt);
      part[threadIdx.x] = dt;               // borrowed until the next barrier
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * K; i += blockDim.x) {
      const int c = i / K, kk = i - c * K;
      const TA* row = xbc + (size_t)(t0 + c) * ld + inner + (size_t)g * K + kk;
      k_s[i] = __fmul_rn(part[c], to_f32(row[0]));
      if (MODE != RC_LOCAL) c_s[i] = to_f32(row[(size_t)G * K]);
    }
    for (int i = threadIdx.x; i < n * RC_COLS; i += blockDim.x) {
      const int c = i / RC_COLS, j = i - c * RC_COLS;
      v_s[i] = (v0 + j < V) ? to_f32(xbc[(size_t)(t0 + c) * ld + (size_t)h * V + v0 + j]) : 0.f;
    }
    __syncthreads();
    if (MODE == RC_LOCAL) {
      // the segment's own state and the product of its decays; nothing is read out
#pragma unroll 2
      for (int c = 0; c < n; ++c) {
        const float vj = v_s[c * RC_COLS + lane], a = a_s[c];
        const float* kc = k_s + c * K + kk0;
        P *= a;
#pragma unroll
        for (int i = 0; i < KPT; ++i)
          if (kk0 + i < K) S[i] = __fmaf_rn(a, S[i], __fmul_rn(kc[i], vj));
      }
      __syncthreads();
      continue;
    }
#pragma unroll 2
    for (int c = 0; c < n; ++c) {
      const float vj = v_s[c * RC_COLS + lane], a = a_s[c];
      const float* kc = k_s + c * K + kk0;
      const float* cc = c_s + c * K + kk0;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        if (kk0 + i < K) {
          S[i] = __fmaf_rn(a, S[i], __fmul_rn(kc[i], vj));
          acc = __fmaf_rn(S[i], cc[i], acc);
        }
      }
      part[(ks * RC_CHUNK + c) * RC_COLS + lane] = acc;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * RC_COLS; i += blockDim.x) {
      const int c = i / RC_COLS, j = i - c * RC_COLS;
      if (v0 + j < V) {
        float total = 0.f;
        for (int w = 0; w < KS; ++w) total += part[(w * RC_CHUNK + c) * RC_COLS + j];
        out[((size_t)(t0 + c) * H + h) * V + v0 + j] = __fmaf_rn(dsk, v_s[i], total);
      }
    }
    __syncthreads();
  }
  if (MODE == RC_LOCAL) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      const int kk = kk0 + i;
      if (kk < K && col_ok) my_s[((size_t)(seg + 1) * K + kk) * V + col] = S[i];
    }
    if (v0 == 0 && threadIdx.x == 0) my_p[seg + 1] = P;
    return;
  }
  if (MODE == RC_JOINED && seg != nseg_s - 1) return;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    if (kk < K && col_ok) st[(size_t)kk * V + col] = S[i];
  }
}

// gated delta rule.  With D = diag(g) S: u = beta (v - D^T k), o = D^T q + (k . q) u,
// S = D + k u^T: the slices' partial sums of D^T k and D^T q meet once per token.  q and k
// are made unit vectors (q also times q_scale) while a chunk is staged.
//
// A token's step is linear in the state, S_t = A_t S_(t-1) + beta_t k_t v_t^T with
// A_t = (I - beta_t k_t k_t^T) diag(g_t), so long prompts are walked in segments side by
// side like the other recurrences, with a matrix where those have a product of decays:
//   local    every segment but a sequence's last is walked from a zero state without
//            outputs (its own state, entry seg + 1 of `scr_s`), and the same walk over the
//            columns of the identity matrix with values of zero gives the product of its
//            A_t (entry seg + 1 of `scr_a`, [K, K]); entry 0 of `scr_s` takes the slot's state.
//   joined   a segment's start state is rebuilt from the entries before it,
//            S <- A_i S + S_i in ascending i, the segment is walked with outputs, and the
//            last segment leaves the state.  Against the whole walk the results differ by
//            rounding only.
template <typename TA, int KPT, int MODE>
__global__ void __launch_bounds__(RC_COLS * 8)
delta_recurrence_kernel(const TA* __restrict__ q, long long ldq, const TA* __restrict__ k,
                        long long ldk, const TA* __restrict__ v, long long ldv,
                        const TA* __restrict__ beta_raw, long long ldb,
                        const float* __restrict__ decay, float* __restrict__ state,
                        const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                        float* __restrict__ out, int H, int HK, int K, int V, int KS,
                        float unit_eps, float q_scale, int seg_len, int nseg,
                        float* __restrict__ scr_s, float* __restrict__ scr_a) {
  extern __shared__ __align__(16) float sm[];
  // rows of KP = KS * KPT entries: the entries from K on stay zero, so that every slice
  // reads its KPT entries of a token as whole float4 without asking where the head ends
  const int KP = KS * KPT;
  float* q_s = sm;                          // [RC_CHUNK][KP]
  float* k_s = q_s + RC_CHUNK * KP;         // [RC_CHUNK][KP]
  float* g_s = k_s + RC_CHUNK * KP;         // [RC_CHUNK][KP]
  float* v_s = g_s + RC_CHUNK * KP;         // [RC_CHUNK][RC_COLS]
  float* b_s = v_s + RC_CHUNK * RC_COLS;    // [RC_CHUNK] beta
  float* kq_s = b_s + RC_CHUNK;             // [RC_CHUNK] k . q
  float* part = kq_s + RC_CHUNK;            // [2][KS][2][RC_COLS]
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31, ks = threadIdx.x >> 5;
  const int vtiles = (V + RC_COLS - 1) / RC_COLS;
  const int tiles = vtiles + (MODE == RC_LOCAL ? (K + RC_COLS - 1) / RC_COLS : 0);
  const int seg = blockIdx.x / tiles, tile = blockIdx.x % tiles;
  const bool a_tile = tile >= vtiles;       // columns of the segment's transition matrix
  const int v0 = (a_tile ? tile - vtiles : tile) * RC_COLS, h = blockIdx.y, s = blockIdx.z;
  const int col = v0 + lane;
  const bool col_ok = col < (a_tile ? K : V);
  const int j = h / (H / HK);
  const int seq_begin = cu_q[s], seq_end = cu_q[s + 1];
  if (seq_end <= seq_begin) return;
  const int nseg_s = MODE == RC_WHOLE ? 1 : (seq_end - seq_begin + seg_len - 1) / seg_len;
  if (seg >= nseg_s) return;
  const int t_begin = MODE == RC_WHOLE ? seq_begin : seq_begin + seg * seg_len;
  const int t_end = MODE == RC_WHOLE ? seq_end : min(seq_end, t_begin + seg_len);
  float* st = state + ((size_t)state_slot[s] * H + h) * K * V;
  float* my_s = scr_s + ((size_t)s * H + h) * nseg * K * V;
  float* my_a = scr_a + ((size_t)s * H + h) * nseg * K * K;
  const bool walks = MODE != RC_LOCAL || seg < nseg_s - 1;
  const int kk0 = ks * KPT;
  float S[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    const bool ok = kk < K && col_ok;
    if (MODE == RC_WHOLE) {
      S[i] = ok ? st[(size_t)kk * V + col] : 0.f;
    } else if (MODE == RC_LOCAL) {
      if (!a_tile && seg == 0 && ok) my_s[(size_t)kk * V + col] = st[(size_t)kk * V + col];
      S[i] = (a_tile && ok && kk == col) ? 1.f : 0.f;
    } else {
      S[i] = ok ? my_s[(size_t)kk * V + col] : 0.f;
    }
  }
  if (MODE == RC_JOINED) {
    float* x_s = q_s;                       // [K][RC_COLS]: the state's columns, all slices'
    for (int e = 1; e <= seg; ++e) {
#pragma unroll
      for (int i = 0; i < KPT; ++i)
        if (kk0 + i < K) x_s[(kk0 + i) * RC_COLS + lane] = S[i];
      __syncthreads();
      const float* A = my_a + (size_t)e * K * K;
      float acc[KPT];
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const int kk = kk0 + i;
        acc[i] = (kk < K && col_ok) ? my_s[((size_t)e * K + kk) * V + col] : 0.f;
      }
      if ((K & 3) == 0) {                   // four entries of a row per load, same order of sums
        for (int jj = 0; jj < K; jj += 4) {
          const float x0 = x_s[jj * RC_COLS + lane], x1 = x_s[(jj + 1) * RC_COLS + lane];
          const float x2 = x_s[(jj + 2) * RC_COLS + lane], x3 = x_s[(jj + 3) * RC_COLS + lane];
#pragma unroll
          for (int i = 0; i < KPT; ++i)
            if (kk0 + i < K) {
              const float4 a = *reinterpret_cast<const float4*>(A + (size_t)(kk0 + i) * K + jj);
              acc[i] = fmaf(a.w, x3, fmaf(a.z, x2, fmaf(a.y, x1, fmaf(a.x, x0, acc[i]))));
            }
        }
      } else {
        for (int jj = 0; jj < K; ++jj) {
          const float x = x_s[jj * RC_COLS + lane];
#pragma unroll
          for (int i = 0; i < KPT; ++i)
            if (kk0 + i < K) acc[i] = fmaf(A[(size_t)(kk0 + i) * K + jj], x, acc[i]);
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < KPT; ++i) S[i] = acc[i];
    }
  }
  if (!walks) return;
  if (KP > K) {
    const int pad = KP - K;
    for (int i = threadIdx.x; i < RC_CHUNK * pad; i += blockDim.x) {
      const int at = (i / pad) * KP + K + i % pad;
      q_s[at] = 0.f;
      k_s[at] = 0.f;
      g_s[at] = 0.f;
    }
  }
  int buf = 0;
  const int st_c = threadIdx.x / K, st_k = threadIdx.x % K;
  const int step_c = blockDim.x / K, step_k = blockDim.x % K;
  for (int t0 = t_begin; t0 < t_end; t0 += RC_CHUNK) {
    const int n = min(RC_CHUNK, t_end - t0);
    // thread i takes entries i, i + blockDim.x, ... of the chunk's [n][K]; its (token, entry)
    // advances by a fixed step, so no division runs per entry
    for (int c = st_c, kk = st_k; c < n;) {
      const size_t t = (size_t)(t0 + c);
      if (MODE != RC_LOCAL) q_s[c * KP + kk] = to_f32(q[t * ldq + (size_t)j * K + kk]);
      k_s[c * KP + kk] = to_f32(k[t * ldk + (size_t)j * K + kk]);
      g_s[c * KP + kk] = decay[(t * H + h) * K + kk];
      c += step_c;
      kk += step_k;
      if (kk >= K) {
        kk -= K;
        ++c;
      }
    }
    for (int i = threadIdx.x; i < n * RC_COLS; i += blockDim.x) {
      const int c = i / RC_COLS, jj = i - c * RC_COLS;
      v_s[i] = (!a_tile && v0 + jj < V)
                   ? to_f32(v[(size_t)(t0 + c) * ldv + (size_t)h * V + v0 + jj]) : 0.f;
    }
    if (threadIdx.x < n) {
      const float z = to_f32(beta_raw[(size_t)(t0 + threadIdx.x) * ldb + h]);
      b_s[threadIdx.x] = 1.0f / (1.0f + expf(-z));
    }
    __syncthreads();
    // unit vectors: one warp a token; sums over lanes in strides of 32, then a shuffle tree
    for (int c = ks; c < n; c += KS) {
      float sq = 0.f, sk = 0.f;
      for (int kk = lane; kk < K; kk += 32) {
        if (MODE != RC_LOCAL) sq = fmaf(q_s[c * KP + kk], q_s[c * KP + kk], sq);
        sk = fmaf(k_s[c * KP + kk], k_s[c * KP + kk], sk);
      }
      const float iq = MODE != RC_LOCAL ? q_scale / sqrtf(warp_sum(sq) + unit_eps) : 0.f;
      const float ik = 1.0f / sqrtf(warp_sum(sk) + unit_eps);
      float dot = 0.f;
      for (int kk = lane; kk < K; kk += 32) {
        const float kv = k_s[c * KP + kk] * ik;
        k_s[c * KP + kk] = kv;
        if (MODE != RC_LOCAL) {
          const float qq = q_s[c * KP + kk] * iq;
          q_s[c * KP + kk] = qq;
          dot = fmaf(qq, kv, dot);
        }
      }
      if (MODE != RC_LOCAL) {
        dot = warp_sum(dot);
        if (lane == 0) kq_s[c] = dot;
      }
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float4* g4 = reinterpret_cast<const float4*>(g_s + c * KP + kk0);
      const float4* k4 = reinterpret_cast<const float4*>(k_s + c * KP + kk0);
      const float4* q4 = reinterpret_cast<const float4*>(q_s + c * KP + kk0);
      float pk = 0.f, pq = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; i += 4) {
        const float4 gv = g4[i / 4], kv = k4[i / 4];
        const float gc[4] = {gv.x, gv.y, gv.z, gv.w}, kc[4] = {kv.x, kv.y, kv.z, kv.w};
        float qc[4] = {0.f, 0.f, 0.f, 0.f};
        if (MODE != RC_LOCAL) {
          const float4 qv = q4[i / 4];
          qc[0] = qv.x, qc[1] = qv.y, qc[2] = qv.z, qc[3] = qv.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          S[i + e] = __fmul_rn(gc[e], S[i + e]);
          pk = __fmaf_rn(S[i + e], kc[e], pk);
          if (MODE != RC_LOCAL) pq = __fmaf_rn(S[i + e], qc[e], pq);
        }
      }
      float* pb = part + (size_t)buf * KS * 2 * RC_COLS;
      pb[(ks * 2 + 0) * RC_COLS + lane] = pk;
      if (MODE != RC_LOCAL) pb[(ks * 2 + 1) * RC_COLS + lane] = pq;
      __syncthreads();
      float kd = 0.f, qd = 0.f;
      for (int w = 0; w < KS; ++w) kd += pb[(w * 2 + 0) * RC_COLS + lane];
      if (MODE != RC_LOCAL && ks == 0)      // the first slice writes the outputs
        for (int w = 0; w < KS; ++w) qd += pb[(w * 2 + 1) * RC_COLS + lane];
      const float u = __fmul_rn(b_s[c], v_s[c * RC_COLS + lane] - kd);
#pragma unroll
      for (int i = 0; i < KPT; i += 4) {
        const float4 kv = k4[i / 4];
        S[i] = __fmaf_rn(kv.x, u, S[i]);
        S[i + 1] = __fmaf_rn(kv.y, u, S[i + 1]);
        S[i + 2] = __fmaf_rn(kv.z, u, S[i + 2]);
        S[i + 3] = __fmaf_rn(kv.w, u, S[i + 3]);
      }
      if (MODE != RC_LOCAL && ks == 0 && col_ok)
        out[((size_t)(t0 + c) * H + h) * V + col] = __fmaf_rn(kq_s[c], u, qd);
      buf ^= 1;
    }
    __syncthreads();
  }
  if (MODE == RC_LOCAL) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      const int kk = kk0 + i;
      if (kk < K && col_ok) {
        if (a_tile) my_a[((size_t)(seg + 1) * K + kk) * K + col] = S[i];
        else my_s[((size_t)(seg + 1) * K + kk) * V + col] = S[i];
      }
    }
    return;
  }
  if (MODE == RC_JOINED && seg != nseg_s - 1) return;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kk0 + i;
    if (kk < K && col_ok) st[(size_t)kk * V + col] = S[i];
  }
}

IX_API int ix_delta_recurrence_max_dim() { return 8 * 64; }

static inline int rc_slices(int K) { return K > 32 ? 8 : (K > 8 ? 4 : 1); }

// Floats of scratch the segmented state-space walk needs.
IX_API long long ix_ssd_recurrence_scratch_floats(int S, int H, int K, int V, int nseg) {
  return nseg <= 1 ? 0 : (long long)S * H * nseg * ((long long)K * V + 1);
}

// seg_len, nseg: 0, 1 for the walk from end to end; otherwise every sequence is cut into
// segments of seg_len tokens (nseg covers the longest) and `scratch` holds
// ix_ssd_recurrence_scratch_floats floats.
IX_API int ix_ssd_recurrence(const void* xbc, long long ld, const void* dt_raw, long long ld_dt,
                             int dtype, const float* dt_bias, const float* a_log,
                             const float* d_skip, float* state, const int* cu_q,
                             const int* state_slot, float* out, int S, int H, int V, int K, int G,
                             int seg_len, int nseg, float* scratch, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (H <= 0 || V <= 0 || K <= 0 || G <= 0 || H % G || K > 8 * 64 || H > 65535 || S > 65535)
    return IX_ERR_SIZE;
  if (ld < (long long)H * V + 2LL * G * K || ld_dt < H) return IX_ERR_SIZE;
  if (nseg < 1 || (nseg > 1 && (seg_len <= 0 || !scratch))) return IX_ERR_SIZE;
  const int KS = rc_slices(K);
  const int kpt = (K + KS - 1) / KS;
  const size_t smem = ((size_t)2 * RC_CHUNK * K + RC_CHUNK * RC_COLS + RC_CHUNK +
                       (size_t)KS * RC_CHUNK * RC_COLS) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  const int vtiles = (V + RC_COLS - 1) / RC_COLS;
  dim3 grid(vtiles * nseg, H, S), block(RC_COLS * KS);
  float* scr_s = scratch;
  float* scr_p = scratch ? scratch + (size_t)S * H * nseg * K * V : nullptr;
#define SSD_ONE(KPT, MODE)                                                                   \
  IX_DISPATCH_DTYPE(dtype, TA, {                                                             \
    auto kern = ssd_recurrence_kernel<TA, KPT, MODE>;                                        \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    ix_launch(kern, grid, block, smem, stream, (const TA*)xbc, ld, (const TA*)dt_raw, ld_dt, \
              dt_bias, a_log, d_skip, state, cu_q, state_slot, out, H, V, K, G, KS, seg_len, \
              nseg, scr_s, scr_p);                                                           \
  })
#define SSD_GO(KPT)                                                                          \
  do {                                                                                       \
    if (nseg <= 1) {                                                                         \
      SSD_ONE(KPT, RC_WHOLE);                                                                \
    } else {                                                                                 \
      SSD_ONE(KPT, RC_LOCAL);                                                                \
      SSD_ONE(KPT, RC_JOINED);                                                               \
    }                                                                                        \
  } while (0)
  if (kpt <= 8) SSD_GO(8);
  else if (kpt <= 16) SSD_GO(16);
  else if (kpt <= 32) SSD_GO(32);
  else SSD_GO(64);
#undef SSD_GO
#undef SSD_ONE
  return ix_launch_status();
}

template <typename TA, int KPT>
static int dr_resident(int mode, size_t smem, int threads) {
  int n = 0;
  if (mode == RC_LOCAL) {
    auto kern = delta_recurrence_kernel<TA, KPT, RC_LOCAL>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem);
  } else {
    auto kern = delta_recurrence_kernel<TA, KPT, RC_JOINED>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem);
  }
  return n;
}

// Segments for a step whose longest sequence brings max_q_len tokens: as many as keep each
// of the two passes within the blocks the device holds at once (a second, nearly empty
// round of blocks would double a pass), none shorter than 64 tokens.  Returns the number
// of segments and sets *seg_len; 1 and 0 when the sequences are walked from end to end.
IX_API int ix_delta_recurrence_segments(int dtype, int S, int H, int K, int V, int max_q_len,
                                        int min_tokens, int max_segments, int* seg_len) {
  *seg_len = 0;
  if (S <= 0 || H <= 0 || K <= 0 || V <= 0 || K > 8 * 64 || max_q_len < min_tokens) return 1;
  const int KS = rc_slices(K);
  const int kpt = (K + KS - 1) / KS;
  const int KPT = kpt <= 8 ? 8 : kpt <= 16 ? 16 : kpt <= 32 ? 32 : 64;
  const size_t smem = ((size_t)3 * RC_CHUNK * KS * KPT + RC_CHUNK * RC_COLS + 2 * RC_CHUNK +
                       (size_t)2 * KS * 2 * RC_COLS) * sizeof(float);
  int dev = 0, sms = 0, local = 0, joined = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
#define DR_OCC(KK)                                                                           \
  IX_DISPATCH_DTYPE(dtype, TA, {                                                             \
    local = dr_resident<TA, KK>(RC_LOCAL, smem, RC_COLS * KS);                               \
    joined = dr_resident<TA, KK>(RC_JOINED, smem, RC_COLS * KS);                             \
  })
  if (KPT == 8) DR_OCC(8);
  else if (KPT == 16) DR_OCC(16);
  else if (KPT == 32) DR_OCC(32);
  else DR_OCC(64);
#undef DR_OCC
  const long long vtiles = (V + RC_COLS - 1) / RC_COLS, atiles = (K + RC_COLS - 1) / RC_COLS;
  const long long per_joined = (long long)S * H * vtiles;
  const long long per_local = (long long)S * H * (vtiles + atiles);
  long long want = (long long)joined * sms / per_joined;
  if ((long long)local * sms / per_local < want) want = (long long)local * sms / per_local;
  if (want > max_segments) want = max_segments;
  if (want < 2) return 1;
  int len = (int)((max_q_len + want - 1) / want);
  len = (len + RC_CHUNK - 1) / RC_CHUNK * RC_CHUNK;
  if (len < 64) len = 64;
  const int nseg = (max_q_len + len - 1) / len;
  if (nseg <= 1) return 1;
  *seg_len = len;
  return nseg;
}

// Floats of scratch the segmented delta walk needs.
IX_API long long ix_delta_recurrence_scratch_floats(int S, int H, int K, int V, int nseg) {
  return nseg <= 1 ? 0 : (long long)S * H * nseg * ((long long)K * V + (long long)K * K);
}

// seg_len, nseg: 0, 1 for the walk from end to end; otherwise every sequence is cut into
// segments of seg_len tokens (nseg covers the longest) and `scratch` holds
// ix_delta_recurrence_scratch_floats floats.
IX_API int ix_delta_recurrence(const void* q, long long ldq, const void* k, long long ldk,
                               const void* v, long long ldv, const void* beta_raw, long long ldb,
                               int dtype, const float* decay, float* state, const int* cu_q,
                               const int* state_slot, float* out, int S, int H, int HK, int K,
                               int V, float unit_eps, float q_scale, int seg_len, int nseg,
                               float* scratch, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (H <= 0 || HK <= 0 || H % HK || K <= 0 || V <= 0 || K > 8 * 64 || H > 65535 || S > 65535)
    return IX_ERR_SIZE;
  if (ldq < (long long)HK * K || ldk < (long long)HK * K || ldv < (long long)H * V || ldb < H)
    return IX_ERR_SIZE;
  if (nseg < 1 || (nseg > 1 && (seg_len <= 0 || !scratch))) return IX_ERR_SIZE;
  const int KS = rc_slices(K);
  const int kpt = (K + KS - 1) / KS;
  const int kp = KS * (kpt <= 8 ? 8 : kpt <= 16 ? 16 : kpt <= 32 ? 32 : 64);
  const size_t smem = ((size_t)3 * RC_CHUNK * kp + RC_CHUNK * RC_COLS + 2 * RC_CHUNK +
                       (size_t)2 * KS * 2 * RC_COLS) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  const int vtiles = (V + RC_COLS - 1) / RC_COLS, atiles = (K + RC_COLS - 1) / RC_COLS;
  const dim3 block(RC_COLS * KS);
  float* scr_s = scratch;
  float* scr_a = scratch ? scratch + (size_t)S * H * nseg * K * V : nullptr;
#define DR_ONE(KPT, MODE, TILES)                                                             \
  IX_DISPATCH_DTYPE(dtype, TA, {                                                             \
    auto kern = delta_recurrence_kernel<TA, KPT, MODE>;                                      \
    if (smem > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    ix_launch(kern, dim3((TILES) * nseg, H, S), block, smem, stream, (const TA*)q, ldq,      \
              (const TA*)k, ldk, (const TA*)v, ldv, (const TA*)beta_raw, ldb, decay, state,  \
              cu_q, state_slot, out, H, HK, K, V, KS, unit_eps, q_scale, seg_len, nseg,      \
              scr_s, scr_a);                                                                 \
  })
#define DR_GO(KPT)                                                                           \
  do {                                                                                       \
    if (nseg <= 1) {                                                                         \
      DR_ONE(KPT, RC_WHOLE, vtiles);                                                         \
    } else {                                                                                 \
      DR_ONE(KPT, RC_LOCAL, vtiles + atiles);                                                \
      DR_ONE(KPT, RC_JOINED, vtiles);                                                        \
    }                                                                                        \
  } while (0)
  if (kpt <= 8) DR_GO(8);
  else if (kpt <= 16) DR_GO(16);
  else if (kpt <= 32) DR_GO(32);
  else DR_GO(64);
#undef DR_GO
#undef DR_ONE
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// gate + group norm: out = groupnorm(y * silu(z)) * gain.  One block per (token, group).
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const TA* __restrict__ z,
                                        long long ldz, const float* __restrict__ gain,
                                        TA* __restrict__ out, int W, int groups, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x, g = blockIdx.y;
  const int n = W / groups, c0 = g * n;
  const float* yr = y + (size_t)t * W + c0;
  const TA* zr = z + (size_t)t * ldz + c0;
  float sq = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float zz = to_f32(zr[i]);
    const float v = yr[i] * (zz / (1.0f + expf(-zz)));
    sq += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float zz = to_f32(zr[i]);
    const float v = yr[i] * (zz / (1.0f + expf(-zz)));
    out[(size_t)t * W + c0 + i] = from_f32<TA>(v * inv * gain[c0 + i]);
  }
}

// four entries per access (groups of a multiple of four entries, rows on such boundaries);
// against the form above a thread's partial sums run over other entries
template <typename TA>
__global__ void gated_group_norm_vec_kernel(const float* __restrict__ y,
                                            const TA* __restrict__ z, long long ldz,
                                            const float* __restrict__ gain,
                                            TA* __restrict__ out, int W, int groups, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x, g = blockIdx.y;
  const int n = W / groups, c0 = g * n;
  const float* yr = y + (size_t)t * W + c0;
  const TA* zr = z + (size_t)t * ldz + c0;
  float sq = 0.f;
  for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
    const float4 zz = ld4(zr + i), yy = ld4(yr + i);
    const float a = yy.x * (zz.x / (1.0f + expf(-zz.x))), b = yy.y * (zz.y / (1.0f + expf(-zz.y)));
    const float c = yy.z * (zz.z / (1.0f + expf(-zz.z))), d = yy.w * (zz.w / (1.0f + expf(-zz.w)));
    sq += (a * a + b * b) + (c * c + d * d);
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
    const float4 zz = ld4(zr + i), yy = ld4(yr + i), gg = ld4(gain + c0 + i);
    const float a = yy.x * (zz.x / (1.0f + expf(-zz.x))), b = yy.y * (zz.y / (1.0f + expf(-zz.y)));
    const float c = yy.z * (zz.z / (1.0f + expf(-zz.z))), d = yy.w * (zz.w / (1.0f + expf(-zz.w)));
    st4(out + (size_t)t * W + c0 + i,
        make_float4(a * inv * gg.x, b * inv * gg.y, c * inv * gg.z, d * inv * gg.w));
  }
}

static inline bool at_four(const void* p, size_t elem) { return ((uintptr_t)p % (4 * elem)) == 0; }

IX_API int ix_gated_group_norm(const float* y, const void* z, int dtype, long long ldz,
                               const float* gain, void* out, int T, int W, int groups, float eps,
                               cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0 || groups <= 0 || W % groups || ldz < W || groups > 65535) return IX_ERR_SIZE;
  const int n = W / groups;
  const size_t el = dtype == IX_F32 ? 4 : 2;
  const bool vec = n % 4 == 0 && ldz % 4 == 0 && at_four(y, 4) && at_four(gain, 4) &&
                   at_four(z, el) && at_four(out, el);
  const int threads = vec ? (n >= 2048 ? 256 : (n >= 512 ? 128 : 64))
                          : (n >= 1024 ? 256 : (n >= 256 ? 128 : 64));
  IX_DISPATCH_DTYPE(dtype, TA, {
    auto kern = vec ? gated_group_norm_vec_kernel<TA> : gated_group_norm_kernel<TA>;
    ix_launch(kern, dim3(T, groups), dim3(threads), 0, stream, y, (const TA*)z, ldz, gain,
              (TA*)out, W, groups, eps);
  });
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// normed pair mean: out = (l / rms(l) * gl + r / rms(r) * gr) / 2, all fp32.
// ---------------------------------------------------------------------------
template <typename TL>
__global__ void normed_pair_mean_kernel(const TL* __restrict__ l, const TL* __restrict__ r,
                                        const float* __restrict__ gl,
                                        const float* __restrict__ gr, float* __restrict__ out,
                                        int W, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const TL* lr = l + (size_t)t * W;
  const TL* rr = r + (size_t)t * W;
  float sl = 0.f, sr = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float a = to_f32(lr[i]), b = to_f32(rr[i]);
    sl += a * a;
    sr += b * b;
  }
  const float il = 1.0f / sqrtf(block_sum(sl, scratch) / (float)W + eps);
  const float ir = 1.0f / sqrtf(block_sum(sr, scratch) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(size_t)t * W + i] = 0.5f * (to_f32(lr[i]) * il * gl[i] + to_f32(rr[i]) * ir * gr[i]);
}

template <typename TL>
__global__ void normed_pair_mean_vec_kernel(const TL* __restrict__ l, const TL* __restrict__ r,
                                            const float* __restrict__ gl,
                                            const float* __restrict__ gr,
                                            float* __restrict__ out, int W, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const TL* lr = l + (size_t)t * W;
  const TL* rr = r + (size_t)t * W;
  float sl = 0.f, sr = 0.f;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 a = ld4(lr + i), b = ld4(rr + i);
    sl += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
    sr += (b.x * b.x + b.y * b.y) + (b.z * b.z + b.w * b.w);
  }
  const float il = 1.0f / sqrtf(block_sum(sl, scratch) / (float)W + eps);
  const float ir = 1.0f / sqrtf(block_sum(sr, scratch) / (float)W + eps);
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 a = ld4(lr + i), b = ld4(rr + i), ga = ld4(gl + i), gb = ld4(gr + i);
    st4(out + (size_t)t * W + i,
        make_float4(0.5f * (a.x * il * ga.x + b.x * ir * gb.x),
                    0.5f * (a.y * il * ga.y + b.y * ir * gb.y),
                    0.5f * (a.z * il * ga.z + b.z * ir * gb.z),
                    0.5f * (a.w * il * ga.w + b.w * ir * gb.w)));
  }
}

IX_API int ix_normed_pair_mean(const void* l, const void* r, int dtype, const float* gl,
                               const float* gr, float* out, int T, int W, float eps,
                               cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0) return IX_ERR_SIZE;
  const size_t el = dtype == IX_F32 ? 4 : 2;
  const bool vec = W % 4 == 0 && at_four(l, el) && at_four(r, el) && at_four(gl, 4) &&
                   at_four(gr, 4) && at_four(out, 4);
  const int threads = vec ? (W >= 4096 ? 512 : (W >= 1024 ? 256 : 128))
                          : (W >= 2048 ? 512 : (W >= 512 ? 256 : 128));
  IX_DISPATCH_DTYPE(dtype, TL, {
    auto kern = vec ? normed_pair_mean_vec_kernel<TL> : normed_pair_mean_kernel<TL>;
    ix_launch(kern, dim3(T), dim3(threads), 0, stream, (const TL*)l, (const TL*)r, gl, gr, out,
              W, eps);
  });
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// relu squared; table routing; rows times a constant.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void relu_squared_kernel(const TA* __restrict__ x, TA* __restrict__ out, size_t n) {
  IX_PDL_WAIT();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_f32(x[i]), 0.f);
    out[i] = from_f32<TA>(v * v);
  }
}

IX_API int ix_relu_squared(const void* x, void* out, int dtype, long long n,
                           cudaStream_t stream) {
  if (n <= 0) return IX_OK;
  const long long want = (n + 255) / 256;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  IX_DISPATCH_DTYPE(dtype, TA,
                    ix_launch(relu_squared_kernel<TA>, dim3(blocks), dim3(256), 0, stream,
                              (const TA*)x, (TA*)out, (size_t)n));
  return ix_launch_status();
}

__global__ void table_route_kernel(const int* __restrict__ ids, const int* __restrict__ table,
                                   int* __restrict__ idx, float* __restrict__ wts, int T, int top,
                                   int vocab, int experts) {
  IX_PDL_WAIT();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * top) return;
  const int t = i / top, j = i - t * top;
  const int id = min(max(ids[t], 0), vocab - 1);
  idx[i] = min(max(table[(size_t)id * top + j], 0), experts - 1);
  wts[i] = 1.0f / (float)top;
}

IX_API int ix_table_route(const int* ids, const int* table, int* idx, float* wts, int T, int top,
                          int vocab, int experts, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (top <= 0 || vocab <= 0 || experts <= 0) return IX_ERR_SIZE;
  const int n = T * top;
  ix_launch(table_route_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, table, idx, wts,
            T, top, vocab, experts);
  return ix_launch_status();
}

__global__ void scale_rows_kernel(float* __restrict__ x, float scale, size_t n) {
  IX_PDL_WAIT();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] *= scale;
}

IX_API int ix_scale_rows(float* x, float scale, long long n, cudaStream_t stream) {
  if (n <= 0) return IX_OK;
  const long long want = (n + 255) / 256;
  const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
  ix_launch(scale_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, scale, (size_t)n);
  return ix_launch_status();
}
