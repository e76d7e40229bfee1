// Split-KV attention for decode steps (one query per sequence) with head sizes the tuned
// kernels do not take: any size up to 512, the values' size may differ from the keys', any
// element type, fp32 arithmetic with the accurate expf and tanhf.
//
// The work is bandwidth: the keys of a sequence are split across thread blocks, query heads
// that share a key/value head are handled by the same block (up to G of them), so that a
// key and a value are read once for the group.  A warp takes four keys at a time; its lanes
// stride over the head's entries (entry d of a row belongs to lane d % 32: neighbouring
// lanes read neighbouring addresses whatever the head size), form the partial dot products of
// the block's heads and add them across the warp.  Online softmax per warp and head in
// registers; the warps meet once in shared memory; the block writes an unnormalised partial
// (o, max, sum) per head, or the result when the sequence is not split.  A second small
// kernel merges the partials.  A query's arithmetic depends on its own keys and on the
// number of splits alone.
//
// `keep_first` > 0 keeps the sequence's first keep_first keys visible beside the window: the
// walk goes over them and then over the window, as one range that is split.  `sink` adds
// one to the softmax's denominator (a key of score 0 without a value), where the result
// is normalised: in this kernel when the sequence is not split, else in the merge.
//
// Scratch: partial outputs [S, heads, splits, vd] and (max, sum) [S, heads, splits, 2], fp32.
#include "common.cuh"

#define DA_THREADS 128
#define DA_WARPS 4
#define DA_U 4          // keys a warp handles per iteration

// D: entries of a head per lane (head sizes up to 32 * D); G: query heads per block.
template <typename TA, int D, int G>
__global__ void __launch_bounds__(DA_THREADS)
attn_decode_any_kernel(const TA* __restrict__ q, const TA* __restrict__ kc,
                       const TA* __restrict__ vc, const int* __restrict__ block_table,
                       const int* __restrict__ kv_len, float* __restrict__ part_o,
                       float* __restrict__ part_ml, TA* __restrict__ out, int heads, int kvh,
                       int hd, int vd, int page_size, int maxb, int window, float scale,
                       float softcap, int splits, int keep_first, int sink) {
  extern __shared__ float sm[];
  float* sm_acc = sm;                               // [G][DA_WARPS][vd]
  float* sm_m = sm_acc + (size_t)G * DA_WARPS * vd; // [G][DA_WARPS]
  float* sm_l = sm_m + G * DA_WARPS;                // [G][DA_WARPS]
  IX_PDL_WAIT();
  const int split = blockIdx.x, s = blockIdx.z;
  const int rep = heads / kvh;
  const int per_kv = (rep + G - 1) / G;
  const int kh = blockIdx.y / per_kv;
  const int g0 = (blockIdx.y % per_kv) * G;
  const int gcount = min(G, rep - g0);
  const int h0 = kh * rep + g0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const int len = kv_len[s];
  const int start = window > 0 ? max(0, len - window) : 0;
  // the kept first keys stand, in the walk, directly before the window: walk index j means
  // key j - (start - kept) below `start` and key j from there on
  const int kept = min(keep_first, start);
  const int shift = start - kept;
  const int n = len - shift;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + DA_WARPS * DA_U - 1) / (DA_WARPS * DA_U) * (DA_WARPS * DA_U);
  const int k0 = shift + split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int* bt = block_table + (size_t)s * maxb;

  float qr[G][D], acc[G][D], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < D; ++e) {
      const int d = lane + 32 * e;
      acc[g][e] = 0.f;
      qr[g][e] = (g < gcount && d < hd) ? to_f32(q[((size_t)s * heads + h0 + g) * hd + d]) : 0.f;
    }
  }

  int dk[D], dv[D];
#pragma unroll
  for (int e = 0; e < D; ++e) {
    dk[e] = lane + 32 * e < hd ? lane + 32 * e : 0;
    dv[e] = lane + 32 * e < vd ? lane + 32 * e : 0;
  }
  for (int kb = k0 + warp * DA_U; kb < k1; kb += DA_WARPS * DA_U) {
    const TA* krow[DA_U];
    const TA* vrow[DA_U];
    bool valid[DA_U];
#pragma unroll
    for (int u = 0; u < DA_U; ++u) {
      const int kwalk = kb + u;
      const int kidx = kwalk < start ? kwalk - shift : kwalk;
      valid[u] = kwalk < k1;
      const int page = valid[u] ? bt[kidx / page_size] : 0;
      const size_t row = ((size_t)page * kvh + kh) * page_size + (valid[u] ? kidx % page_size : 0);
      krow[u] = kc + row * hd;
      vrow[u] = vc + row * vd;
    }
    // every load is issued before the first is used: entries past the head's size and keys
    // past the range read a valid address (entry 0; row 0 of page 0) and count as zero
    TA kraw[DA_U][D], vraw[DA_U][D];
#pragma unroll
    for (int u = 0; u < DA_U; ++u)
#pragma unroll
      for (int e = 0; e < D; ++e) kraw[u][e] = krow[u][dk[e]];
#pragma unroll
    for (int u = 0; u < DA_U; ++u)
#pragma unroll
      for (int e = 0; e < D; ++e) vraw[u][e] = vrow[u][dv[e]];
    float kf[DA_U][D], vf[DA_U][D];
#pragma unroll
    for (int u = 0; u < DA_U; ++u)
#pragma unroll
      for (int e = 0; e < D; ++e) {
        kf[u][e] = (valid[u] && lane + 32 * e < hd) ? to_f32(kraw[u][e]) : 0.f;
        vf[u][e] = (valid[u] && lane + 32 * e < vd) ? to_f32(vraw[u][e]) : 0.f;
      }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g >= gcount) break;
      float sc[DA_U];
#pragma unroll
      for (int u = 0; u < DA_U; ++u) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < D; ++e) dot = fmaf(qr[g][e], kf[u][e], dot);
        dot = warp_sum(dot);
        float sv = dot * scale;
        if (softcap > 0.f) sv = softcap * tanhf(sv / softcap);
        sc[u] = valid[u] ? sv : -INFINITY;
      }
      float m_new = m[g];
#pragma unroll
      for (int u = 0; u < DA_U; ++u) m_new = fmaxf(m_new, sc[u]);
      if (m_new == -INFINITY) continue;
      const float corr = expf(m[g] - m_new);      // 0 at the first keys (m = -inf)
      float p[DA_U], psum = 0.f;
#pragma unroll
      for (int u = 0; u < DA_U; ++u) {
        p[u] = expf(sc[u] - m_new);
        psum += p[u];
      }
      l[g] = l[g] * corr + psum;
      m[g] = m_new;
#pragma unroll
      for (int e = 0; e < D; ++e) {
        float a = acc[g][e] * corr;
#pragma unroll
        for (int u = 0; u < DA_U; ++u) a = fmaf(p[u], vf[u][e], a);
        acc[g][e] = a;
      }
    }
  }

  // the warps meet: every lane of a warp holds the same (m, l) and its own entries of o
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (g >= gcount) break;
#pragma unroll
    for (int e = 0; e < D; ++e) {
      const int d = lane + 32 * e;
      if (d < vd) sm_acc[((size_t)g * DA_WARPS + warp) * vd + d] = acc[g][e];
    }
    if (lane == 0) {
      sm_m[g * DA_WARPS + warp] = m[g];
      sm_l[g * DA_WARPS + warp] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < gcount * vd; idx += DA_THREADS) {
    const int g = idx / vd, d = idx - g * vd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DA_WARPS; ++w) M = fmaxf(M, sm_m[g * DA_WARPS + w]);
    float o = 0.f, L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DA_WARPS; ++w) {
        const float mw = sm_m[g * DA_WARPS + w];
        if (mw == -INFINITY) continue;
        const float cw = expf(mw - M);
        o = fmaf(sm_acc[((size_t)g * DA_WARPS + w) * vd + d], cw, o);
        L = fmaf(sm_l[g * DA_WARPS + w], cw, L);
      }
    }
    const size_t hrow = (size_t)s * heads + h0 + g;
    if (splits == 1) {
      if (sink && M != -INFINITY) {
        const float top = fmaxf(M, 0.f);
        const float c = expf(M - top);
        o *= c;
        L = L * c + expf(-top);
      }
      out[hrow * vd + d] = from_f32<TA>(L > 0.f ? o / L : 0.f);
    } else {
      part_o[(hrow * splits + split) * vd + d] = o;
      if (d == 0) {
        part_ml[(hrow * splits + split) * 2] = M;
        part_ml[(hrow * splits + split) * 2 + 1] = L;
      }
    }
  }
}

template <typename TA>
__global__ void attn_decode_any_merge_kernel(const float* __restrict__ part_o,
                                             const float* __restrict__ part_ml,
                                             TA* __restrict__ out, int vd, int splits,
                                             int sink) {
  IX_PDL_WAIT();
  const size_t hrow = blockIdx.x;   // s * heads + h
  const float* ml = part_ml + hrow * splits * 2;
  float M = -INFINITY;
  for (int j = 0; j < splits; ++j) M = fmaxf(M, ml[2 * j]);
  float L = 0.f;
  for (int j = 0; j < splits; ++j)
    if (ml[2 * j] != -INFINITY) L = fmaf(ml[2 * j + 1], expf(ml[2 * j] - M), L);
  float c = 1.f;
  if (sink && M != -INFINITY) {
    const float top = fmaxf(M, 0.f);
    c = expf(M - top);
    L = L * c + expf(-top);
  }
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float o = 0.f;
    for (int j = 0; j < splits; ++j)
      if (ml[2 * j] != -INFINITY)
        o = fmaf(part_o[(hrow * splits + j) * vd + d], expf(ml[2 * j] - M), o);
    out[hrow * vd + d] = from_f32<TA>(L > 0.f ? o * c / L : 0.f);
  }
}

// Query heads a block handles for `rep` heads per key/value head and head sizes up to
// 32 * dpl: as many as share the key/value head, while a thread's registers hold their
// queries and outputs.
static int da_group(int rep, int dpl) {
  int g = 8;
  while (g > 1 && (g * dpl > (dpl >= 16 ? 16 : 32) || g / 2 >= rep)) g /= 2;
  return g;
}

static int da_dpl(int hd, int vd) {
  const int most = hd > vd ? hd : vd;
  return most <= 64 ? 2 : most <= 128 ? 4 : most <= 256 ? 8 : 16;
}

// Splits that fill the multiprocessors about four times over, none shorter than 64 keys.
IX_API int ix_attn_decode_any_splits(int S, int heads, int kvh, int hd, int vd, int max_kv_len) {
  if (S <= 0 || heads <= 0 || kvh <= 0 || heads % kvh) return 1;
  const int rep = heads / kvh;
  const int G = da_group(rep, da_dpl(hd, vd));
  const long long base = (long long)S * kvh * ((rep + G - 1) / G);
  long long want = (4LL * 148 + base - 1) / base;
  const long long most = (max_kv_len + 63) / 64;
  if (want > most) want = most;
  if (want > 64) want = 64;
  return want < 1 ? 1 : (int)want;
}

IX_API int ix_paged_attention_decode_any(const void* q, const void* k_cache, const void* v_cache,
                                         const int* block_table, const int* kv_len, float* part_o,
                                         float* part_ml, void* out, int act_dtype, int S, int heads,
                                         int kvh, int hd, int vd, int page_size, int max_blocks,
                                         int window, float scale, float softcap, int splits,
                                         int keep_first, int sink, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0)
    return IX_ERR_SIZE;
  if (hd <= 0 || hd > 512 || vd <= 0 || vd > 512 || window < 0 || splits < 1 ||
      keep_first < 0)
    return IX_ERR_SIZE;
  if (splits > 1 && (!part_o || !part_ml)) return IX_ERR_SIZE;
  const int rep = heads / kvh;
  const int dpl = da_dpl(hd, vd);
  const int G = da_group(rep, dpl);
  const int per_kv = (rep + G - 1) / G;
  if ((long long)kvh * per_kv > 65535 || S > 65535) return IX_ERR_SIZE;
  dim3 grid(splits, kvh * per_kv, S);
  const size_t smem = ((size_t)G * DA_WARPS * vd + 2 * G * DA_WARPS) * sizeof(float);
#define DA_GO(DD, GG)                                                                          \
  IX_DISPATCH_DTYPE(act_dtype, TA, {                                                           \
    auto kern = attn_decode_any_kernel<TA, DD, GG>;                                            \
    if (smem > 48 * 1024)                                                                      \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    ix_launch(kern, grid, dim3(DA_THREADS), smem, stream, (const TA*)q, (const TA*)k_cache,    \
              (const TA*)v_cache, block_table, kv_len, part_o, part_ml, (TA*)out, heads, kvh,  \
              hd, vd, page_size, max_blocks, window, scale, softcap, splits, keep_first, sink); \
  })
#define DA_D(DD)                                                                               \
  do {                                                                                         \
    if (G == 8) DA_GO(DD, (DD <= 4 ? 8 : 1));                                                  \
    else if (G == 4) DA_GO(DD, (DD <= 8 ? 4 : 1));                                             \
    else if (G == 2) DA_GO(DD, 2);                                                             \
    else DA_GO(DD, 1);                                                                         \
  } while (0)
  if (dpl == 2) DA_D(2);
  else if (dpl == 4) DA_D(4);
  else if (dpl == 8) DA_D(8);
  else DA_D(16);
#undef DA_D
#undef DA_GO
  int rc = ix_launch_status();
  if (rc != 0 || splits == 1) return rc;
  IX_DISPATCH_DTYPE(act_dtype, TA, {
    ix_launch(attn_decode_any_merge_kernel<TA>, dim3(S * heads), dim3(vd >= 128 ? 128 : 64), 0,
              stream, (const float*)part_o, (const float*)part_ml, (TA*)out, vd, splits, sink);
  });
  return ix_launch_status();
}
