// Kernels of decoders whose attention prepares q, k and v between the projection and the
// cache, whose stream starts from a pair of tokens, and whose gated units have biases.
//
//  * ix_embed_pair_norm: stream[t] = rmsnorm(embed[token] + pair[row]) * gain with row =
//    (previous * mul_prev + token * mul_cur) mod buckets, row `buckets` for a sequence's
//    first token; the previous token of a sequence's first token in this step is read
//    from per-request state, which then takes the step's last token of the sequence.
//  * ix_attention_prepare: per token, in this order: RMS norm of the whole q row and of
//    the whole k row with gains (optional); rotation of the first `rot` entries of every
//    q and k head by position * frequency, pairs being neighbours or half a rotation
//    apart, cos and sin times a factor; division of every q and k head by its root mean
//    square (optional); values blended with another layer's, (1 - lambda) v + lambda v0
//    (optional); q written densely, k and v into their pages.
//  * ix_glu_bias_act: act(g + b_g) * (u + b_u) over rows laid out g | u, act the tanh form
//    of gelu or silu.
//  * ix_identity_rows: grouped rows of experts that return their input.
//
// All sums, norms, angles and blends are fp32 with the accurate sincosf, tanhf and expf,
// whatever the element type of the rows; a token's result depends on its own row alone.
#include "common.cuh"
#include "elementwise_vec.cuh"

#define PP_THREADS 256

// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(PP_THREADS)
embed_pair_norm_kernel(const TA* __restrict__ table, const TA* __restrict__ pairs,
                       const float* __restrict__ gain, const int* __restrict__ ids,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                       const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                       int* __restrict__ prev_state, float* __restrict__ out, int H,
                       long long buckets, long long mul_prev, long long mul_cur, float eps) {
  __shared__ float scratch[32];
  __shared__ long long row_sh;
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int tok = ids[t];
  if (threadIdx.x == 0) {
    const int s = seq_of_token[t];
    const int first = cu_q[s];
    long long row = buckets;
    int prev = 0;
    if (t > first) prev = ids[t - 1];
    else prev = prev_state[state_slot[s]];
    if (positions[t] != 0) row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    // the block of a sequence's first token here is the only reader of the state, so it is
    // the one that moves it on, after its read
    if (t == first) prev_state[state_slot[s]] = ids[cu_q[s + 1] - 1];
    row_sh = row;
  }
  __syncthreads();
  const TA* a = table + (size_t)tok * H;
  const TA* b = pairs + (size_t)row_sh * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += PP_THREADS) {
    const float x = to_f32(a[i]) + to_f32(b[i]);
    ss += x * x;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += PP_THREADS) {
    const float x = to_f32(a[i]) + to_f32(b[i]);
    out[(size_t)t * H + i] = x * inv * gain[i];
  }
}

IX_API int ix_embed_pair_norm(const void* table, const void* pairs, int dtype, const float* gain,
                              const int* ids, const int* positions, const int* seq_of_token,
                              const int* cu_q, const int* state_slot, int* prev_state,
                              float* out, int T, int H, long long buckets, long long mul_prev,
                              long long mul_cur, float eps, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return IX_ERR_SIZE;
  IX_DISPATCH_DTYPE(dtype, TA, {
    ix_launch(embed_pair_norm_kernel<TA>, dim3(T), dim3(PP_THREADS), 0, stream,
              (const TA*)table, (const TA*)pairs, gain, ids, positions, seq_of_token, cu_q,
              state_slot, prev_state, out, H, buckets, mul_prev, mul_cur, eps);
  });
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// Threads of a block of the preparation kernel: with 128 a multiprocessor holds sixteen
// blocks, so that all tokens of a 2,048-token step are in flight at once and one block's
// barriers are covered by the others' loads.
#define PA_THREADS 128

// One block per token.  The q and k parts of the row are held in shared memory as fp32
// from the first read to the last write.  VEC (bfloat16 rows whose parts start on 16-byte
// marks and whose head sizes are multiples of 8): the row is read and everything is written
// in 16-byte accesses; the arithmetic and its order are the same.
template <typename TA, bool VEC>
__global__ void __launch_bounds__(PA_THREADS)
attention_prepare_kernel(const TA* __restrict__ qkv, long long ld, const int* __restrict__ positions,
                         const float* __restrict__ freq, float magnitude, int rot, int interleaved,
                         int heads, int kvh, int hd, int vd, const float* __restrict__ q_gain,
                         const float* __restrict__ k_gain, float eps, int head_unit,
                         const TA* __restrict__ earlier, long long ld_earlier,
                         const float* __restrict__ lam, const int* __restrict__ slots,
                         TA* __restrict__ q_out, TA* __restrict__ k_cache,
                         TA* __restrict__ v_cache, int page_size, TA* __restrict__ k_dense,
                         TA* __restrict__ v_dense) {
  extern __shared__ float row[];            // [dq + dk], then cos and sin of the pairs [rot]
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int dq = heads * hd, dk = kvh * hd, dv = kvh * vd;
  const TA* src = qkv + (size_t)t * ld;
  const int tid = threadIdx.x;
  float* turn = row + dq + dk;              // cos of pair i, then sin of pair i
  if (rot > 0) {                            // once per token: every head turns by the same angles
    const float pos = (float)positions[t];
    for (int i = tid; i < (rot >> 1); i += PA_THREADS) {
      float sn, cs;
      sincosf(pos * freq[i], &sn, &cs);
      turn[i] = cs * magnitude;
      turn[(rot >> 1) + i] = sn * magnitude;
    }
  }
  float sq = 0.f, sk = 0.f;
  if constexpr (VEC) {
    const uint4* src8 = reinterpret_cast<const uint4*>(src);
    for (int c = tid; c < (dq + dk) >> 3; c += PA_THREADS) {
      float x[8];
      bf8_to_f32(src8[c], x);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        row[8 * c + e] = x[e];
        ss += x[e] * x[e];
      }
      if (8 * c < dq) sq += ss; else sk += ss;
    }
  } else {
    for (int i = tid; i < dq + dk; i += PA_THREADS) {
      const float x = to_f32(src[i]);
      row[i] = x;
      if (i < dq) sq += x * x; else sk += x * x;
    }
  }
  if (q_gain) {
    // both sums in one meeting of the block: warp w's pair sits at scratch[2 w], [2 w + 1]
    {
      const int lane = tid & 31, warp = tid >> 5;
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      if (lane == 0) {
        scratch[2 * warp] = sq;
        scratch[2 * warp + 1] = sk;
      }
      __syncthreads();
      sq = sk = 0.f;
      for (int w = 0; w < PA_THREADS / 32; ++w) {     // ascending warps: a fixed order
        sq += scratch[2 * w];
        sk += scratch[2 * w + 1];
      }
    }
    const float iq = 1.0f / sqrtf(sq / (float)dq + eps);
    const float ik = 1.0f / sqrtf(sk / (float)dk + eps);
    for (int i = tid; i < dq + dk; i += PA_THREADS)
      row[i] = i < dq ? row[i] * iq * q_gain[i] : row[i] * ik * k_gain[i - dq];
  }
  __syncthreads();
  if (rot > 0) {
    const int half = rot >> 1;
    for (int idx = tid; idx < (heads + kvh) * half; idx += PA_THREADS) {
      const int h = idx / half, i = idx - h * half;
      const float cs = turn[i], sn = turn[half + i];
      float* v = row + (size_t)h * hd;
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float x = v[a], y = v[b];
      v[a] = x * cs - y * sn;
      v[b] = y * cs + x * sn;
    }
    __syncthreads();
  }
  if (head_unit) {
    const int lane = tid & 31, warp = tid >> 5;
    for (int h = warp; h < heads + kvh; h += PA_THREADS / 32) {
      float* v = row + (size_t)h * hd;
      float ss = 0.f;
      for (int d = lane; d < hd; d += 32) ss += v[d] * v[d];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      for (int d = lane; d < hd; d += 32) v[d] *= inv;
    }
    __syncthreads();
  }
  const int slot = slots ? slots[t] : -1;
  TA* qo = q_out + (size_t)t * dq;
  const bool cached = k_cache != nullptr && slot >= 0;
  const size_t page = cached ? slot / page_size : 0, off = cached ? slot % page_size : 0;
  if constexpr (VEC) {
    for (int c = tid; c < dq >> 3; c += PA_THREADS)
      reinterpret_cast<uint4*>(qo)[c] = f32_to_bf8(row + 8 * c);
    for (int c = tid; c < dk >> 3; c += PA_THREADS) {
      const int i = 8 * c, kh = i / hd, d = i - kh * hd;
      const uint4 val = f32_to_bf8(row + dq + i);
      if (cached)
        *reinterpret_cast<uint4*>(k_cache + ((page * kvh + kh) * page_size + off) * hd + d) = val;
      if (k_dense) *reinterpret_cast<uint4*>(k_dense + (size_t)t * dk + i) = val;
    }
    const float m = earlier ? lam[0] : 0.f;
    for (int c = tid; c < dv >> 3; c += PA_THREADS) {
      const int i = 8 * c, kh = i / vd, d = i - kh * vd;
      uint4 val = *reinterpret_cast<const uint4*>(src + dq + dk + i);
      if (earlier) {
        float v[8], e8[8];
        bf8_to_f32(val, v);
        bf8_to_f32(*reinterpret_cast<const uint4*>(earlier + (size_t)t * ld_earlier + i), e8);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (1.0f - m) * v[e] + m * e8[e];
        val = f32_to_bf8(v);
      }
      if (cached)
        *reinterpret_cast<uint4*>(v_cache + ((page * kvh + kh) * page_size + off) * vd + d) = val;
      if (v_dense) *reinterpret_cast<uint4*>(v_dense + (size_t)t * dv + i) = val;
    }
  } else {
  for (int i = tid; i < dq; i += PA_THREADS) qo[i] = from_f32<TA>(row[i]);
  for (int i = tid; i < dk; i += PA_THREADS) {
    const int kh = i / hd, d = i - kh * hd;
    const TA val = from_f32<TA>(row[dq + i]);
    if (cached) k_cache[((page * kvh + kh) * page_size + off) * hd + d] = val;
    if (k_dense) k_dense[(size_t)t * dk + i] = val;
  }
  const float m = earlier ? lam[0] : 0.f;
  for (int i = tid; i < dv; i += PA_THREADS) {
    float v = to_f32(src[dq + dk + i]);
    if (earlier) v = (1.0f - m) * v + m * to_f32(earlier[(size_t)t * ld_earlier + i]);
    const int kh = i / vd, d = i - kh * vd;
    const TA val = from_f32<TA>(v);
    if (cached) v_cache[((page * kvh + kh) * page_size + off) * vd + d] = val;
    if (v_dense) v_dense[(size_t)t * dv + i] = val;
  }
  }
}

IX_API int ix_attention_prepare_max_row() { return (200 * 1024) / 4; }

IX_API int ix_attention_prepare(const void* qkv, long long ld, int dtype, const int* positions,
                                const float* freq, float magnitude, int rot, int interleaved,
                                int heads, int kvh, int hd, int vd, const float* q_gain,
                                const float* k_gain, float eps, int head_unit,
                                const void* earlier, long long ld_earlier, const float* lam,
                                const int* slots, void* q_out, void* k_cache, void* v_cache,
                                int page_size, void* k_dense, void* v_dense, int T,
                                cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || hd <= 0 || vd <= 0 || rot < 0 || rot > hd || (rot & 1) ||
      page_size <= 0)
    return IX_ERR_SIZE;
  if ((q_gain == nullptr) != (k_gain == nullptr) || (rot > 0 && !freq) || (earlier && !lam) ||
      (k_cache && (!v_cache || !slots)))
    return IX_ERR_SIZE;
  const size_t smem = ((size_t)(heads + kvh) * hd + rot) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  const bool vec =
      dtype == IX_BF16 && hd % 8 == 0 && vd % 8 == 0 && ld % 8 == 0 && ld_earlier % 8 == 0 &&
      (((uintptr_t)qkv | (uintptr_t)earlier | (uintptr_t)q_out | (uintptr_t)k_cache |
        (uintptr_t)v_cache | (uintptr_t)k_dense | (uintptr_t)v_dense) & 15) == 0;
#define PP_PREPARE(TA, VEC)                                                                     \
  do {                                                                                          \
    auto kern = attention_prepare_kernel<TA, VEC>;                                              \
    if (smem > 48 * 1024) {                                                                     \
      cudaError_t e =                                                                           \
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                      \
    }                                                                                           \
    ix_launch(kern, dim3(T), dim3(PA_THREADS), smem, stream, (const TA*)qkv, ld, positions,     \
              freq, magnitude, rot, interleaved, heads, kvh, hd, vd, q_gain, k_gain, eps,       \
              head_unit, (const TA*)earlier, ld_earlier, lam, slots, (TA*)q_out, (TA*)k_cache,  \
              (TA*)v_cache, page_size, (TA*)k_dense, (TA*)v_dense);                             \
  } while (0)
  if (vec) PP_PREPARE(bf16, true);
  else if (dtype == IX_BF16) PP_PREPARE(bf16, false);
  else if (dtype == IX_F32) PP_PREPARE(float, false);
  else return IX_ERR_DTYPE;
#undef PP_PREPARE
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
__device__ __forceinline__ float pp_act(float g, int silu) {
  if (silu) return g / (1.0f + expf(-g));
  return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

template <typename TA>
__global__ void glu_bias_act_kernel(const TA* __restrict__ gu, const float* __restrict__ bias,
                                    TA* __restrict__ out, long long total, int I, int silu) {
  IX_PDL_WAIT();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int j = (int)(idx - t * I);
    float g = to_f32(gu[t * 2 * I + j]);
    float u = to_f32(gu[t * 2 * I + I + j]);
    if (bias) {
      g += bias[j];
      u += bias[I + j];
    }
    out[idx] = from_f32<TA>(pp_act(g, silu) * u);
  }
}

// bf16 rows in 8-element chunks: 16-byte loads of gate and up, one 16-byte store
__global__ void __launch_bounds__(256)
glu_bias_act_bf16_vec_kernel(const uint4* __restrict__ gu, const float* __restrict__ bias,
                             uint4* __restrict__ out, unsigned total_chunks,
                             unsigned chunks_per_row, int silu) {
  IX_PDL_WAIT();
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_chunks; i += stride) {
    const unsigned t = i / chunks_per_row, c = i - t * chunks_per_row;
    const uint4 gr = gu[(size_t)t * 2 * chunks_per_row + c];
    const uint4 ur = gu[(size_t)t * 2 * chunks_per_row + chunks_per_row + c];
    float g[8], u[8], o[8];
    bf8_to_f32(gr, g);
    bf8_to_f32(ur, u);
    if (bias) {
      const float4* bg = reinterpret_cast<const float4*>(bias + 8 * c);
      const float4* bu = reinterpret_cast<const float4*>(bias + 8 * (chunks_per_row + c));
      const float4 g0 = bg[0], g1 = bg[1], u0 = bu[0], u1 = bu[1];
      g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w;
      g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
      u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w;
      u[4] += u1.x; u[5] += u1.y; u[6] += u1.z; u[7] += u1.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = pp_act(g[e], silu) * u[e];
    out[i] = f32_to_bf8(o);
  }
}

IX_API int ix_glu_bias_act(const void* gu, const float* bias, void* out, int dtype, int T, int I,
                           int silu, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (I <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * I;
  if (dtype == IX_BF16 && I % 8 == 0 && total / 8 < (1LL << 31) &&
      (((uintptr_t)gu | (uintptr_t)out | (uintptr_t)bias) & 15) == 0) {
    const unsigned chunks = (unsigned)(total / 8);
    long long blocks = (chunks + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ix_launch(glu_bias_act_bf16_vec_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
              (const uint4*)gu, bias, (uint4*)out, chunks, (unsigned)(I / 8), silu);
    return ix_launch_status();
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  IX_DISPATCH_DTYPE(dtype, TA, {
    ix_launch(glu_bias_act_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream,
              (const TA*)gu, bias, (TA*)out, total, I, silu);
  });
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// y[r] = x[rows[r]] for the grouped rows r of the router's outputs from `first` on (experts
// that return their input); offsets has `outputs + 1` entries.
template <typename TA>
__global__ void identity_rows_kernel(const TA* __restrict__ x, const int* __restrict__ rows,
                                     const int* __restrict__ offsets, int first, int outputs,
                                     TA* __restrict__ y, int H) {
  IX_PDL_WAIT();
  const int lo = offsets[first], hi = offsets[outputs];
  for (int r = lo + blockIdx.x; r < hi; r += gridDim.x) {
    const TA* src = x + (size_t)rows[r] * H;
    TA* dst = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

IX_API int ix_identity_rows(const void* x, const int* rows, const int* offsets, int first,
                            int outputs, void* y, int dtype, int A, int H, cudaStream_t stream) {
  if (A <= 0 || outputs <= first) return IX_OK;
  if (H <= 0 || first < 0) return IX_ERR_SIZE;
  const int blocks = A < 148 * 8 ? A : 148 * 8;
  IX_DISPATCH_DTYPE(dtype, TA, {
    ix_launch(identity_rows_kernel<TA>, dim3(blocks), dim3(256), 0, stream, (const TA*)x, rows,
              offsets, first, outputs, (TA*)y, H);
  });
  return ix_launch_status();
}
