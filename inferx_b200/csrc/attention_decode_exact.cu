// Split-KV attention for decode steps (one query per sequence) on the tensor cores, for
// decoders that want their attention weights in 32-bit arithmetic, with the options of a
// windowed layer that keeps a sequence's first keys and of a softmax with one added to its
// denominator.
//
// The walk is the one of the cp.async-fed kernel in attention_decode.cu: a block's four
// warps share 64-key tiles streamed through a ring in shared memory (each key row fetched
// from its page with 16-byte copies, so any page size works), each warp takes 16 keys of a
// tile, S = Q K^T and O += P V by mma.sync.m16n8k16 with the up to 16 query heads of a
// key/value head on the M side, an online softmax per warp, the warps merged through shared
// memory, partials (o, max, sum) per split merged by a second kernel.  What differs:
//  * a softmax weight enters its product with the values as two bfloat16 terms, its
//    rounding and the rounding of what that left over, both into the same fp32
//    accumulator: 16 bits of the weight instead of 8 (scores are exact products of
//    bfloat16 numbers summed in fp32; maxima, exponentials and sums are fp32);
//    With at most 8 query heads a key/value head (FOLD) rows 8..15 of the 16-row tile are
//    idle, and the second term of head r rides there: row r + 8 of P holds what rounding
//    row r left over, one product serves both, and row r + 8 of O is added to row r at the
//    end.  Otherwise the second term is a second product.
//  * value heads of a size of their own (64 or 128, as the keys');
//  * `keep_first`: the sequence's first keep_first keys stay visible beside the window;
//    the walk goes over them and then over the window as one range that is split;
//  * `sink`: one is added to the denominator where the result is normalised.
//
// Scratch: partial outputs [S, heads, splits, vd] and (max, sum) [S, heads, splits, 2],
// fp32; maxima are in units of log2 (scores are pre-multiplied by log2 e).
#include "common.cuh"

#define DX_THREADS 128
#define DX_WARPS 4
#define DX_BN 64
#define DX_STAGES 2

__device__ __forceinline__ float dx_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void dx_cp16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void dx_ldsm(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dx_ldsm_t(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dx_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int CH> __device__ __forceinline__ int dx_swz(int r, int c) {
  return (r * CH + (c ^ (r & 7))) * 16;
}
__device__ __forceinline__ unsigned dx_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int HD, int VD, bool FOLD>
__global__ void __launch_bounds__(DX_THREADS)
attn_decode_exact_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                         const bf16* __restrict__ vc, const int* __restrict__ block_table,
                         const int* __restrict__ kv_len, float* __restrict__ part_o,
                         float* __restrict__ part_ml, bf16* __restrict__ out, int heads, int kvh,
                         int page_size, int page_shift, int maxb, int window, float scale_log2e,
                         int splits, int keep_first, int sink) {
  constexpr int CH = HD / 8, CHV = VD / 8, KS = HD / 16, DT = VD / 8;
  constexpr int K_TILE = DX_BN * HD * 2, V_TILE = DX_BN * VD * 2;
  extern __shared__ __align__(128) unsigned char dsm[];
  unsigned char* Qs = dsm;                                   // [16][HD]
  unsigned char* Ks = Qs + 16 * HD * 2;                      // [STAGES][64][HD]
  unsigned char* Vs = Ks + DX_STAGES * K_TILE;               // [STAGES][64][VD]
  __shared__ float sm_m[DX_WARPS][16];
  __shared__ float sm_l[DX_WARPS][16];
  IX_PDL_WAIT();

  const int split = blockIdx.x, s = blockIdx.z;
  const int rep = heads / kvh;
  const int row_groups = (rep + 15) / 16;
  const int kh = blockIdx.y / row_groups;
  const int qrow0 = (blockIdx.y % row_groups) * 16;
  const int rows_valid = min(16, rep - qrow0);
  const int h0 = kh * rep + qrow0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int len = kv_len[s];
  const int start = window > 0 ? max(0, len - window) : 0;
  // the kept first keys stand, in the walk, directly before the window: walk index j means
  // key j - shift below `start` and key j from there on
  const int kept = min(keep_first, start);
  const int shift = start - kept;
  const int n = len - shift;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + DX_BN - 1) / DX_BN * DX_BN;
  const int k0 = shift + split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int n_tiles = k1 > k0 ? (k1 - k0 + DX_BN - 1) / DX_BN : 0;
  const int* bt = block_table + (size_t)s * maxb;

  for (int idx = tid; idx < 16 * CH; idx += DX_THREADS) {
    const int r = idx / CH, c = idx - r * CH;
    const bool ok = r < rows_valid;
    dx_cp16(Qs + dx_swz<CH>(r, c), q + ((size_t)s * heads + h0 + (ok ? r : 0)) * HD + c * 8, ok);
  }
  auto load_kv = [&](int it) {
    if (it < n_tiles) {
      const int stage = it % DX_STAGES;
      const int kbase = k0 + it * DX_BN;
      unsigned char* kd = Ks + stage * K_TILE;
      unsigned char* vd = Vs + stage * V_TILE;
      if (CH == CHV) {        // equal sizes: a row's place is worked out once for both
        for (int idx = tid; idx < DX_BN * CH; idx += DX_THREADS) {
          const int r = idx / CH, c = idx - r * CH;
          const int kw = kbase + r;
          const bool ok = kw < k1;
          size_t off = 0;
          if (ok) {
            const int kp = kw < start ? kw - shift : kw;
            const int pi = page_shift >= 0 ? (kp >> page_shift) : (kp / page_size);
            const int po = page_shift >= 0 ? (kp & (page_size - 1)) : (kp % page_size);
            off = (((size_t)bt[pi] * kvh + kh) * page_size + po) * HD + c * 8;
          }
          dx_cp16(kd + dx_swz<CH>(r, c), kc + off, ok);
          dx_cp16(vd + dx_swz<CH>(r, c), vc + off, ok);
        }
      } else
      for (int idx = tid; idx < DX_BN * (CH + CHV); idx += DX_THREADS) {
        const bool is_v = idx >= DX_BN * CH;
        const int j = is_v ? idx - DX_BN * CH : idx;
        // CH and CHV are powers of two (8 or 16): the compiler divides by shifting
        const int r = is_v ? j / CHV : j / CH, c = is_v ? j - r * CHV : j - r * CH;
        const int kw = kbase + r;
        const bool ok = kw < k1;
        size_t row = 0;
        if (ok) {
          const int kp = kw < start ? kw - shift : kw;
          // page sizes are powers of two nearly always: a shift then, not a division
          const int pi = page_shift >= 0 ? (kp >> page_shift) : (kp / page_size);
          const int po = page_shift >= 0 ? (kp & (page_size - 1)) : (kp % page_size);
          row = ((size_t)bt[pi] * kvh + kh) * page_size + po;
        }
        if (is_v) dx_cp16(vd + dx_swz<CHV>(r, c), vc + row * VD + c * 8, ok);
        else dx_cp16(kd + dx_swz<CH>(r, c), kc + row * HD + c * 8, ok);
      }
    }
    asm volatile("cp.async.commit_group;");
  };
  load_kv(0);

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  unsigned qf[KS][4];

  for (int it = 0; it < n_tiles; ++it) {
    load_kv(it + 1);
    asm volatile("cp.async.wait_group 1;");
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < KS; ++kk)
        dx_ldsm(qf[kk], Qs + dx_swz<CH>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
    }
    const int stage = it % DX_STAGES;
    const unsigned char* kt = Ks + stage * K_TILE;
    const unsigned char* vt = Vs + stage * V_TILE;
    const int kw = k0 + it * DX_BN + warp * 16;      // first key of this warp's 16
    if (kw < k1) {
      float sc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        unsigned b[4];
        dx_ldsm(b, kt + dx_swz<CH>(warp * 16 + (lane >> 4) * 8 + (lane & 7),
                                   kk * 2 + ((lane >> 3) & 1)));
        dx_mma(sc[0], qf[kk], b[0], b[1]);
        dx_mma(sc[1], qf[kk], b[2], b[3]);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int kp = kw + j * 8 + 2 * t + (c & 1);
          const float v = kp < k1 ? sc[j][c] * scale_log2e : -INFINITY;
          sc[j][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = dx_exp2(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
      // (FOLD: rows 8..15 of O belong to rows 0..7 and are rescaled with them)
#pragma unroll
      for (int j = 0; j < DT; ++j) {
        o[j][0] *= corr[0]; o[j][1] *= corr[0];
        o[j][2] *= corr[FOLD ? 0 : 1]; o[j][3] *= corr[FOLD ? 0 : 1];
      }
      unsigned pf[4], pl[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = dx_exp2(sc[j][0] - m_use[0]);
        const float p1 = dx_exp2(sc[j][1] - m_use[0]);
        const float p2 = dx_exp2(sc[j][2] - m_use[1]);
        const float p3 = dx_exp2(sc[j][3] - m_use[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        const __nv_bfloat162 ha = __floats2bfloat162_rn(p0, p1), hb = __floats2bfloat162_rn(p2, p3);
        const float2 fa = __bfloat1622float2(ha), fb = __bfloat1622float2(hb);
        pf[j * 2 + 0] = *reinterpret_cast<const unsigned*>(&ha);
        if (FOLD) {
          pf[j * 2 + 1] = dx_pack(p0 - fa.x, p1 - fa.y);      // row g + 8: the rest of row g
        } else {
          pf[j * 2 + 1] = *reinterpret_cast<const unsigned*>(&hb);
          pl[j * 2 + 0] = dx_pack(p0 - fa.x, p1 - fa.y);
          pl[j * 2 + 1] = dx_pack(p2 - fb.x, p3 - fb.y);
        }
      }
#pragma unroll
      for (int jd = 0; jd < DT; jd += 2) {
        unsigned b[4];
        dx_ldsm_t(b, vt + dx_swz<CHV>(warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7),
                                      jd + (lane >> 4)));
        dx_mma(o[jd], pf, b[0], b[1]);
        dx_mma(o[jd + 1], pf, b[2], b[3]);
        if (!FOLD) {
          dx_mma(o[jd], pl, b[0], b[1]);
          dx_mma(o[jd + 1], pl, b[2], b[3]);
        }
      }
    }
    __syncthreads();   // the stage may be refilled
  }
  asm volatile("cp.async.wait_group 0;");
  __syncthreads();

  // merge the four warps (each saw different keys); stage memory is free now
  float* sm_o = reinterpret_cast<float*>(Ks);     // [DX_WARPS][16][VD], inside Ks + Vs
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (t == 0) {
    sm_m[warp][g] = m_run[0];     sm_l[warp][g] = l_run[0];
    sm_m[warp][g + 8] = m_run[1]; sm_l[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = j * 8 + 2 * t;
    if (FOLD) {            // the second terms' sums join the first terms'
      o[j][0] += o[j][2];
      o[j][1] += o[j][3];
    }
    sm_o[(warp * 16 + g) * VD + d] = o[j][0];
    sm_o[(warp * 16 + g) * VD + d + 1] = o[j][1];
    sm_o[(warp * 16 + g + 8) * VD + d] = o[j][2];
    sm_o[(warp * 16 + g + 8) * VD + d + 1] = o[j][3];
  }
  __syncthreads();
  for (int idx = tid; idx < rows_valid * VD; idx += DX_THREADS) {
    const int r = idx / VD, d = idx - r * VD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DX_WARPS; ++w) M = fmaxf(M, sm_m[w][r]);
    float ov = 0.f, L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DX_WARPS; ++w) {
        const float cw = dx_exp2(sm_m[w][r] - M);   // exp2(-inf) = 0 for idle warps
        ov += sm_o[(w * 16 + r) * VD + d] * cw;
        L += sm_l[w][r] * cw;
      }
    }
    const size_t hrow = (size_t)s * heads + h0 + r;
    if (splits == 1) {
      if (sink && M != -INFINITY) {        // one more term, 2^(0 - max), in the denominator
        const float top = fmaxf(M, 0.f);
        const float c = dx_exp2(M - top);
        ov *= c;
        L = L * c + dx_exp2(-top);
      }
      out[hrow * VD + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
    } else {
      part_o[(hrow * splits + split) * VD + d] = ov;
      if (d == 0) {
        part_ml[(hrow * splits + split) * 2] = M;
        part_ml[(hrow * splits + split) * 2 + 1] = L;
      }
    }
  }
}

__global__ void attn_decode_exact_merge_kernel(const float* __restrict__ part_o,
                                               const float* __restrict__ part_ml,
                                               bf16* __restrict__ out, int vd, int splits,
                                               int sink) {
  IX_PDL_WAIT();
  const size_t hrow = blockIdx.x;   // s * heads + h
  const float* ml = part_ml + hrow * splits * 2;
  float M = -INFINITY;
  for (int j = 0; j < splits; ++j) M = fmaxf(M, ml[2 * j]);
  float L = 0.f;
  for (int j = 0; j < splits; ++j)
    if (ml[2 * j] != -INFINITY) L += ml[2 * j + 1] * dx_exp2(ml[2 * j] - M);
  float c = 1.f;
  if (sink && M != -INFINITY) {
    const float top = fmaxf(M, 0.f);
    c = dx_exp2(M - top);
    L = L * c + dx_exp2(-top);
  }
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float o = 0.f;
    for (int j = 0; j < splits; ++j)
      if (ml[2 * j] != -INFINITY)
        o += part_o[(hrow * splits + j) * vd + d] * dx_exp2(ml[2 * j] - M);
    out[hrow * vd + d] = __float2bfloat16_rn(L > 0.f ? o * c / L : 0.f);
  }
}

template <int HD, int VD>
static int launch_decode_exact(const void* q, const void* kc, const void* vc, const int* bt,
                               const int* kv_len, float* part_o, float* part_ml, void* out, int S,
                               int heads, int kvh, int page_size, int maxb, int window,
                               float scale, int splits, int keep_first, int sink,
                               cudaStream_t stream) {
  const int rep = heads / kvh;
  const float sl2 = scale * 1.4426950408889634f;
  const int smem = 16 * HD * 2 + DX_STAGES * DX_BN * (HD + VD) * 2;
  dim3 grid(splits, kvh * ((rep + 15) / 16), S);
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
#define DX_LAUNCH(FOLD_)                                                                        \
  do {                                                                                          \
    auto kern = attn_decode_exact_kernel<HD, VD, FOLD_>;                                        \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                         smem);                                                 \
    if (e != cudaSuccess) return (int)e;                                                        \
    ix_launch(kern, grid, dim3(DX_THREADS), smem, stream, (const bf16*)q, (const bf16*)kc,      \
              (const bf16*)vc, bt, kv_len, part_o, part_ml, (bf16*)out, heads, kvh, page_size,  \
              page_shift, maxb, window, sl2, splits, keep_first, sink);                         \
  } while (0)
  if (rep <= 8) DX_LAUNCH(true);
  else DX_LAUNCH(false);
#undef DX_LAUNCH
  int rc = ix_launch_status();
  if (rc != 0 || splits == 1) return rc;
  ix_launch(attn_decode_exact_merge_kernel, dim3(S * heads), dim3(VD >= 128 ? 128 : 64), 0,
            stream, (const float*)part_o, (const float*)part_ml, (bf16*)out, VD, splits, sink);
  return ix_launch_status();
}

IX_API int ix_paged_attention_decode_exact_applies(int hd, int vd) {
  return (hd == 64 || hd == 128) && (vd == 64 || vd == 128);
}

// q [S, heads, hd], out [S, heads, vd], caches [pages, kvh, page_size, hd or vd], bfloat16.
IX_API int ix_paged_attention_decode_exact(const void* q, const void* k_cache,
                                           const void* v_cache, const int* block_table,
                                           const int* kv_len, float* part_o, float* part_ml,
                                           void* out, int S, int heads, int kvh, int hd, int vd,
                                           int page_size, int max_blocks, int window, float scale,
                                           int splits, int keep_first, int sink,
                                           cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0 ||
      window < 0 || keep_first < 0 || splits < 1 || !(scale > 0.f))
    return IX_ERR_SIZE;
  if (splits > 1 && (!part_o || !part_ml)) return IX_ERR_SIZE;
  if ((long long)kvh * ((heads / kvh + 15) / 16) > 65535 || S > 65535) return IX_ERR_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return IX_ERR_ALIGN;
#define DX_GO(H_, V_)                                                                         \
  if (hd == H_ && vd == V_)                                                                   \
    return launch_decode_exact<H_, V_>(q, k_cache, v_cache, block_table, kv_len, part_o,      \
                                       part_ml, out, S, heads, kvh, page_size, max_blocks,    \
                                       window, scale, splits, keep_first, sink, stream);
  DX_GO(64, 64)
  DX_GO(64, 128)
  DX_GO(128, 64)
  DX_GO(128, 128)
#undef DX_GO
  return IX_ERR_UNSUPPORTED;
}
