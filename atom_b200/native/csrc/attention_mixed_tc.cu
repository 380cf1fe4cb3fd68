// Causal attention over the paged cache whose heads see one another's scores (the formulas stand in
// attention_mixed.cu), in bfloat16 on the tensor cores, compiled for one set of sizes:
//   -DATOM_MH_NH (query heads) -DATOM_MH_NKV (kv heads) -DATOM_MH_DK (key size) -DATOM_MH_DV (value size).
//
// A CTA of 16 warps takes a tile of 16 consecutive tokens of one request with ALL heads, because mixing the
// heads needs every head's score of a (query, key) pair at once, and walks the keys in chunks of 64:
//   1. per kv head: its 64 keys go to shared memory (cp.async, the next load under way while this one is used); S_h = Q_h K^T for the heads of its group on mma.sync
//      (m16n8k16, 32-bit sums), times scale * temperature of the row, plus the distance bias, to shared
//      memory in 32-bit;
//   2. warp r owns row r: it takes the row's raw scores of all heads into registers, forms every head's
//      mixed score as a 32-bit sum over heads, masks, and keeps the running maximum and sum per (head, row);
//      the weights exp(s - m) are left in shared memory as TWO bfloat16 numbers, p = hi + lo, so that the
//      product with the values sees 16 bits of their mantissa;
//   3. per kv head: its 64 values go to shared memory; O_h = O_h * correction + (P_hi + P_lo) V on mma.sync.
//      The output tiles (head, 16 columns) of a kv head's group are dealt out to the warps, which keep them
//      in registers over all chunks.
// With few tokens in the step the keys of a tile are shared out among `nsplit` CTAs, which leave maximum,
// sum and unnormalised output per (token, head) in the scratch array of attention_mixed.cu's merge kernel.
#include "common.cuh"

#if !defined(ATOM_MH_NH) || !defined(ATOM_MH_NKV) || !defined(ATOM_MH_DK) || !defined(ATOM_MH_DV)
#error "compile with -DATOM_MH_NH= -DATOM_MH_NKV= -DATOM_MH_DK= -DATOM_MH_DV="
#endif

namespace atom {
namespace mixtc {

constexpr int NH = ATOM_MH_NH, NKV = ATOM_MH_NKV, DK = ATOM_MH_DK, DV = ATOM_MH_DV;
constexpr int GROUP = NH / NKV;
constexpr int BM = 16, BN = 64, WARPS = 16, THREADS = WARPS * 32;
constexpr int LDQ = DK + 8;                              // bf16 elements per row of Q in shared memory
constexpr int LDKV = (DK > DV ? DK : DV) + 8;            // ... of the keys' / values' buffer
constexpr int LDR = 72;                                  // floats per (head, row) of raw scores = 288 bytes,
                                                         // later 72 bf16 of P_hi and 72 bf16 of P_lo
constexpr int QK_UNITS = GROUP * (BN / 16);              // (head of the group, 16 keys) per kv head
constexpr int PV_UNITS = GROUP * (DV / 16);              // (head of the group, 16 value columns) per kv head
constexpr int TPG = (PV_UNITS + WARPS - 1) / WARPS;      // output tiles of a warp per kv head
constexpr int MAX_THR = 256;
static_assert(NH % NKV == 0 && DK % 16 == 0 && DV % 16 == 0, "sizes");
static_assert(NKV * TPG * 8 <= 64, "output tiles of a warp exceed its registers");

constexpr size_t smem_bytes(bool mix) {
  return sizeof(__nv_bfloat16) * ((size_t)NH * BM * LDQ + (size_t)2 * BN * LDKV) + sizeof(float) * ((size_t)NH * BM * LDR) +
         sizeof(float) * (mix ? NH * NH : 0) + sizeof(float) * (3 * NH * BM + BM) + sizeof(int) * (2 * BN + MAX_THR) +
         sizeof(short) * 128;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared without passing through registers; !valid: 16 zero bytes, nothing is read.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ int distance_row(int n, int half, const int* thr, int n_thr) {
  if (n < half) return n;
  int b = 0;
  for (int k = 0; k < n_thr; ++k) b += (thr[k] <= n) ? 1 : 0;
  return half + b;
}

// Reduces N values per lane (N a power of two up to 16) over the warp with N - 1 + (5 - log2 N) shuffles instead of
// 5 N: in every halving step a lane hands over the half of its values that its partner keeps.  Afterwards lane L
// holds, in v[0], the warp's total of element (L >> (5 - log2 N)) & (N - 1).
template <int N, bool IS_MAX>
__device__ __forceinline__ float reduce_many(float (&v)[N], int lane) {
  int off = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      const float got = __shfl_xor_sync(0xffffffffu, send, off);
      v[i] = IS_MAX ? fmaxf(keep, got) : keep + got;
    }
    off >>= 1;
  }
  float t = v[0];
  for (; off > 0; off >>= 1) {
    const float got = __shfl_xor_sync(0xffffffffu, t, off);
    t = IS_MAX ? fmaxf(t, got) : t + got;
  }
  return t;
}

constexpr int NHP = NH <= 1 ? 1 : (NH <= 2 ? 2 : (NH <= 4 ? 4 : (NH <= 8 ? 8 : 16)));      // heads, rounded up to a power of two
constexpr int LOG_NHP = NHP == 1 ? 0 : (NHP == 2 ? 1 : (NHP == 4 ? 2 : (NHP == 8 ? 3 : 4)));
static_assert(NH <= 16, "at most 16 heads");

__global__ void __launch_bounds__(THREADS, 1)
attention_mixed_tc_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q, int64_t q_stride,
                          const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                          const int* __restrict__ block_table, int max_pages, int page_size,
                          const int* __restrict__ positions, const int* __restrict__ cu_q, int num_seqs, float scale,
                          int window, const float* __restrict__ rel, int half, const int* __restrict__ thr, int n_thr,
                          const float* __restrict__ mix, const float* __restrict__ sink, float temp_coef,
                          int temp_every, int nsplit, float* __restrict__ part) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = (__nv_bfloat16*)smem_raw;                  // [NH][16][LDQ]
  __nv_bfloat16* KVs = Qs + NH * BM * LDQ;                       // [2][64][LDKV]: one kv head's keys or values, twice
  float* raw = (float*)(KVs + 2 * BN * LDKV);                    // [NH][16][LDR]
  float* mix_s = raw + NH * BM * LDR;                            // [NH][NH] if mixing
  float* m_s = mix_s + (mix ? NH * NH : 0);                      // [NH][16]
  float* l_s = m_s + NH * BM;
  float* corr_s = l_s + NH * BM;
  float* qscale_s = corr_s + NH * BM;                            // [16]
  int* off_s = (int*)(qscale_s + BM);                            // [2][64] row of a key in the pages, kv head 0
  int* thr_s = off_s + 2 * BN;                                   // [MAX_THR]
  short* bkt_s = (short*)(thr_s + MAX_THR);                      // [128] bias row by (row - column + 63)
  __shared__ int tile_s[3];

  if (threadIdx.x == 0) {          // which tile this CTA has: tiles are numbered request by request
    int b = blockIdx.x, found = -1, first = 0, rows = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int a = cu_q[s], n = cu_q[s + 1] - a;
      const int nt = (n + BM - 1) / BM;
      if (b < nt) {
        found = s;
        first = a + b * BM;
        rows = min(BM, n - b * BM);
        break;
      }
      b -= nt;
    }
    tile_s[0] = found;
    tile_s[1] = first;
    tile_s[2] = rows;
  }
  __syncthreads();
  const int seq = tile_s[0], t0 = tile_s[1], nrows = tile_s[2];
  if (seq < 0) return;
  const int p0 = positions[t0];                                   // the tile's rows have positions p0, p0 + 1, ...
  const int* bt = block_table + (int64_t)seq * max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mat = lane >> 3, r8 = lane & 7;
  const int split = blockIdx.y;

  // ---- prologue: Q, tables, running maximum and sum
  for (int e = threadIdx.x; e < NH * BM * (DK / 8); e += THREADS) {
    const int seg = e % (DK / 8), hr = e / (DK / 8);
    const int r = hr % BM, h = hr / BM;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (int64_t)(t0 + r) * q_stride + h * DK + seg * 8);
    *reinterpret_cast<uint4*>(Qs + (h * BM + r) * LDQ + seg * 8) = v;
  }
  if (mix)
    for (int e = threadIdx.x; e < NH * NH; e += THREADS) mix_s[e] = mix[e];
  for (int e = threadIdx.x; e < n_thr; e += THREADS) thr_s[e] = thr[e];
  for (int e = threadIdx.x; e < NH * BM; e += THREADS) {
    const int h = e / BM;
    m_s[e] = (sink && split == 0) ? sink[h] : -INFINITY;          // the sink counts once: in the first share
    l_s[e] = (sink && split == 0) ? 1.f : 0.f;
  }
  if (threadIdx.x < BM) {
    const int p = p0 + threadIdx.x;
    qscale_s[threadIdx.x] = scale * (temp_every > 0 ? 1.f + temp_coef * logf((float)((p + 1) / temp_every) + 1.f) : 1.f);
  }
  float O[NKV][TPG][2][4];
#pragma unroll
  for (int g = 0; g < NKV; ++g)
#pragma unroll
    for (int s = 0; s < TPG; ++s)
#pragma unroll
      for (int n = 0; n < 2; ++n) O[g][s][n][0] = O[g][s][n][1] = O[g][s][n][2] = O[g][s][n][3] = 0.f;

  int lo = 0, hi = p0 + nrows;
  if (window > 0 && p0 - window + 1 > 0) lo = p0 - window + 1;
  if (nsplit > 1) {
    const int per = ((hi - lo + nsplit - 1) / nsplit + BN - 1) / BN * BN;
    lo += split * per;
    hi = min(hi, lo + per);
  }
  __syncthreads();

  // The keys and values of a chunk come as 2 * NKV loads of one kv head's 64 rows each (K of every kv head, then
  // V of every kv head), through two buffers: while the warps work on one load, the next is on its way.
  int issued = 0, used = 0;
  auto key_rows = [&](int c0_, int* offs) {      // threads 0..63: where chunk c0_'s keys lie
    const int j = c0_ + threadIdx.x;
    int off = -1;
    if (j < hi) {
      const int pg = bt[j / page_size];
      off = pg * NKV * page_size + (j % page_size);
    }
    offs[threadIdx.x] = off;
  };
  auto issue = [&](int c0_, int i, const int* offs) {
    __nv_bfloat16* dst = KVs + (issued & 1) * BN * LDKV;
    if (c0_ < hi) {
      if (i < NKV) {
        for (int e = threadIdx.x; e < BN * (DK / 8); e += THREADS) {
          const int seg = e % (DK / 8), key = e / (DK / 8);
          const int off = offs[key];
          cp_async16(dst + key * LDKV + seg * 8,
                     off >= 0 ? k_pages + ((int64_t)off + (int64_t)i * page_size) * DK + seg * 8 : k_pages, off >= 0);
        }
      } else {
        for (int e = threadIdx.x; e < BN * (DV / 8); e += THREADS) {
          const int seg = e % (DV / 8), key = e / (DV / 8);
          const int off = offs[key];
          cp_async16(dst + key * LDKV + seg * 8,
                     off >= 0 ? v_pages + ((int64_t)off + (int64_t)(i - NKV) * page_size) * DV + seg * 8 : v_pages, off >= 0);
        }
      }
    }
    cp_async_commit();
    ++issued;
  };
  if (threadIdx.x < BN) key_rows(lo, off_s);
  __syncthreads();
  issue(lo, 0, off_s);

  int ci = 0;
  for (int c0 = lo; c0 < hi; c0 += BN, ++ci) {
    const int* cur = off_s + (ci & 1) * BN;
    int* nxt = off_s + ((ci + 1) & 1) * BN;
    // ---- where the next chunk's keys lie, and the bias row of every distance that occurs in this chunk
    if (threadIdx.x < BN) {
      key_rows(c0 + BN, nxt);
    } else if (rel && threadIdx.x >= 64 && threadIdx.x < 64 + BM + BN - 1) {
      const int dlt = threadIdx.x - 64;                           // row - column + 63
      const int n = (p0 - c0) + dlt - (BN - 1);
      bkt_s[dlt] = (short)(n < 0 ? 0 : distance_row(n, half, thr_s, n_thr));
    }
    __syncthreads();

    // ---- 1. raw scores of every head
#pragma unroll 1
    for (int g = 0; g < NKV; ++g) {
      issue(c0, g + 1, cur);                                      // the next kv head's keys, or the first one's values
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* Ks = KVs + (used & 1) * BN * LDKV;
      ++used;
      for (int u = warp; u < QK_UNITS; u += WARPS) {
        const int hq = u / (BN / 16), kb = u % (BN / 16);
        const int h = g * GROUP + hq;
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const __nv_bfloat16* qbase = Qs + (h * BM + (mat & 1) * 8 + r8) * LDQ + (mat >> 1) * 8;
        const __nv_bfloat16* kbase = Ks + (kb * 16 + (mat >> 1) * 8 + r8) * LDKV + (mat & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, qbase + ks * 16);
          ldmatrix_x4(b, kbase + ks * 16);
          mma_bf16(s[0], a, b[0], b[1]);
          mma_bf16(s[1], a, b[2], b[3]);
        }
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = (lane >> 2) + (e >= 2 ? 8 : 0);
            const int col = kb * 16 + n * 8 + 2 * (lane & 3) + (e & 1);
            float val = s[n][e] * qscale_s[row];
            if (rel) val += rel[(int)bkt_s[row - col + (BN - 1)] * NH + h];
            raw[(h * BM + row) * LDR + col] = val;
          }
      }
      __syncthreads();
    }

    // ---- 2. mixing, mask, running softmax: warp r has row r
    {
      constexpr int OWNER_SHIFT = 5 - LOG_NHP;                    // lane L answers for head (L >> OWNER_SHIFT) & (NHP - 1)
      const int r = warp;
      const int pr = p0 + r;
      const int j0 = c0 + lane, j1 = j0 + 32;
      bool ok0 = r < nrows && j0 < hi && j0 <= pr, ok1 = r < nrows && j1 < hi && j1 <= pr;
      if (window > 0) {
        ok0 = ok0 && j0 > pr - window;
        ok1 = ok1 && j1 > pr - window;
      }
      float mx[NHP];
      {
        float x0[NH], x1[NH];
#pragma unroll
        for (int g = 0; g < NH; ++g) {
          x0[g] = raw[(g * BM + r) * LDR + lane];
          x1[g] = raw[(g * BM + r) * LDR + lane + 32];
        }
        __syncwarp();
        // the mixed scores go back to the row's place in shared memory; the largest of this lane's two per head stays
#pragma unroll
        for (int h = 0; h < NHP; ++h) {
          float s0 = -INFINITY, s1 = -INFINITY;
          if (h < NH) {
            if (mix) {
              s0 = 0.f;
              s1 = 0.f;
#pragma unroll
              for (int g = 0; g < NH; ++g) {
                const float w = mix_s[(h < NH ? h : 0) * NH + g];
                s0 = fmaf(w, x0[g], s0);
                s1 = fmaf(w, x1[g], s1);
              }
            } else {
              s0 = x0[h < NH ? h : 0];
              s1 = x1[h < NH ? h : 0];
            }
            s0 = ok0 ? s0 : -INFINITY;
            s1 = ok1 ? s1 : -INFINITY;
            raw[(h * BM + r) * LDR + lane] = s0;
            raw[(h * BM + r) * LDR + lane + 32] = s1;
          }
          mx[h] = fmaxf(s0, s1);
        }
      }
      const float row_max = reduce_many<NHP, true>(mx, lane);
      const int own = (lane >> OWNER_SHIFT) & (NHP - 1);          // the head this lane answers for
      const bool owner = own < NH && (lane & ((1 << OWNER_SHIFT) - 1)) == 0;
      float m_old_own = 0.f, m_use_own = 0.f;
      if (owner) {
        m_old_own = m_s[own * BM + r];
        const float m_new = fmaxf(m_old_own, row_max);
        m_use_own = (m_new == -INFINITY) ? 0.f : m_new;
        m_s[own * BM + r] = m_new;
      }
      __syncwarp();
      float psum[NHP];
#pragma unroll
      for (int h = 0; h < NHP; ++h) {
        psum[h] = 0.f;
        if (h < NH) {
          const float m_new = m_s[h * BM + r];
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          const float p0f = expf(raw[(h * BM + r) * LDR + lane] - m_use);        // exp(-inf) = 0 for masked keys
          const float p1f = expf(raw[(h * BM + r) * LDR + lane + 32] - m_use);
          psum[h] = p0f + p1f;
          __syncwarp();                                            // (all lanes have read the row's scores)
          __nv_bfloat16* ph = reinterpret_cast<__nv_bfloat16*>(raw + (h * BM + r) * LDR);
          const __nv_bfloat16 h0 = __float2bfloat16_rn(p0f), h1 = __float2bfloat16_rn(p1f);
          ph[lane] = h0;
          ph[lane + 32] = h1;
          ph[LDR + lane] = __float2bfloat16_rn(p0f - __bfloat162float(h0));
          ph[LDR + lane + 32] = __float2bfloat16_rn(p1f - __bfloat162float(h1));
        }
      }
      const float row_sum = reduce_many<NHP, false>(psum, lane);
      if (owner) {
        const float corr = expf(m_old_own - m_use_own);
        corr_s[own * BM + r] = corr;
        l_s[own * BM + r] = l_s[own * BM + r] * corr + row_sum;
      }
    }
    __syncthreads();

    // ---- 3. O = O * correction + P V
#pragma unroll
    for (int g = 0; g < NKV; ++g) {
      if (g + 1 < NKV)
        issue(c0, NKV + g + 1, cur);                              // the next kv head's values
      else
        issue(c0 + BN, 0, nxt);                                   // the next chunk's first keys
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* Vs = KVs + (used & 1) * BN * LDKV;
      ++used;
#pragma unroll
      for (int s = 0; s < TPG; ++s) {
        const int u = warp + WARPS * s;
        if (u < PV_UNITS) {
          const int hq = u / (DV / 16), db = u % (DV / 16);
          const int h = g * GROUP + hq;
          const float c_lo = corr_s[h * BM + (lane >> 2)], c_hi = corr_s[h * BM + (lane >> 2) + 8];
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            O[g][s][n][0] *= c_lo;
            O[g][s][n][1] *= c_lo;
            O[g][s][n][2] *= c_hi;
            O[g][s][n][3] *= c_hi;
          }
          const __nv_bfloat16* pbase = reinterpret_cast<const __nv_bfloat16*>(raw + (h * BM + (mat & 1) * 8 + r8) * LDR) + (mat >> 1) * 8;
          const __nv_bfloat16* vbase = Vs + ((mat & 1) * 8 + r8) * LDKV + (mat >> 1) * 8 + db * 16;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t ah[4], al[4], b[4];
            ldmatrix_x4(ah, pbase + kk * 16);
            ldmatrix_x4(al, pbase + LDR + kk * 16);
            ldmatrix_x4_trans(b, vbase + kk * 16 * LDKV);
            mma_bf16(O[g][s][0], ah, b[0], b[1]);
            mma_bf16(O[g][s][1], ah, b[2], b[3]);
            mma_bf16(O[g][s][0], al, b[0], b[1]);
            mma_bf16(O[g][s][1], al, b[2], b[3]);
          }
        }
      }
      __syncthreads();
    }
  }

  cp_async_wait<0>();
  // ---- epilogue
  constexpr int n_out = NH * DV;
  if (nsplit > 1) {
    for (int e = threadIdx.x; e < NH * BM; e += THREADS) {
      const int h = e / BM, r = e % BM;
      if (r < nrows) {
        float* pt = part + ((int64_t)(t0 + r) * nsplit + split) * (n_out + 2 * NH);
        pt[h] = m_s[e];
        pt[NH + h] = l_s[e];
      }
    }
  }
#pragma unroll
  for (int g = 0; g < NKV; ++g)
#pragma unroll
    for (int s = 0; s < TPG; ++s) {
      const int u = warp + WARPS * s;
      if (u < PV_UNITS) {
        const int hq = u / (DV / 16), db = u % (DV / 16);
        const int h = g * GROUP + hq;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int half_ = 0; half_ < 2; ++half_) {
            const int row = (lane >> 2) + half_ * 8;
            const int col = h * DV + db * 16 + n * 8 + 2 * (lane & 3);
            if (row < nrows) {
              const float a = O[g][s][n][2 * half_], b = O[g][s][n][2 * half_ + 1];
              if (nsplit > 1) {
                float* pt = part + ((int64_t)(t0 + row) * nsplit + split) * (n_out + 2 * NH) + 2 * NH + col;
                pt[0] = a;
                pt[1] = b;
              } else {
                const float inv = 1.f / l_s[h * BM + row];
                *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(t0 + row) * n_out + col) = __floats2bfloat162_rn(a * inv, b * inv);
              }
            }
          }
      }
    }
}

}  // namespace mixtc
}  // namespace atom

ATOM_EXPORT int atom_mixtc_sizes(int* nh, int* nkv, int* dk, int* dv) {
  *nh = atom::mixtc::NH;
  *nkv = atom::mixtc::NKV;
  *dk = atom::mixtc::DK;
  *dv = atom::mixtc::DV;
  return ATOM_OK;
}

ATOM_EXPORT int atom_mixtc_set_option(int key, int value) { return atom::set_option(key, value); }

// Shapes as atom_attention_mixed (attention_mixed.cu); cu_q: [num_seqs + 1] first token row of every request;
// tiles: an upper bound on the number of 16-row tiles, e.g. ceil(T / 16) + num_seqs.  With nsplit > 1 the
// caller runs the merge kernel afterwards.
ATOM_EXPORT int atom_attention_mixed_tc(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                        const void* v_pages, const int* block_table, int max_pages, int page_size,
                                        const int* positions, const int* cu_q, int num_seqs, int tiles, float scale,
                                        int window, const float* rel, int half, const int* thr, int n_thr,
                                        const float* mix, const float* sink, float temp_coef, int temp_every,
                                        int nsplit, float* part, cudaStream_t stream) {
  using namespace atom::mixtc;
  if (tiles <= 0) return ATOM_OK;
  if (n_thr > MAX_THR || nsplit < 1 || nsplit > 65535 || (nsplit > 1 && part == nullptr) || page_size <= 0 ||
      (q_stride % 8) != 0 || ((uintptr_t)q % 16) != 0 || ((uintptr_t)k_pages % 16) != 0 || ((uintptr_t)v_pages % 16) != 0)
    return ATOM_ERR_ARG;
  const size_t smem = smem_bytes(mix != nullptr);
  if (smem_bytes(true) > 226 * 1024) return ATOM_ERR_ARG;      // (the kernel has a few static bytes of its own)
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_mixed_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes(true)) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
  atom::launch_pdl(attention_mixed_tc_kernel, dim3(tiles, nsplit), dim3(THREADS), smem, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                   block_table, max_pages, page_size, positions, cu_q, num_seqs, scale, window, rel, half, thr, n_thr,
                   mix, sink, temp_coef, temp_every, nsplit, part);
  return atom::check_launch();
}
