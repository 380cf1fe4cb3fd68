// Attention over a cached latent on the tensor cores (bfloat16; see latent.cu for the mechanism and the plain
// kernel).  Because every head reads the same row [c | kr] per key, the heads of a token are rows of one
// product: a CTA owns 64 query rows = a few consecutive tokens of one request x a group of heads, and walks the
// keys its tokens may see in tiles of 32:
//   1. the tile's rows come into shared memory once (cp.async, two buffers): they are the K operand of the
//      scores AND, in their first R columns, the V operand of the output;
//   2. S[64 x 32] = Q K^T on mma.sync m16n8k16 (each warp two 16 x 8 tiles over all R + rd columns), 32-bit
//      sums to shared memory;
//   3. warp w owns rows 8w .. 8w + 7: scale, window and causal mask, running maximum and sum per row in 32-bit,
//      the weights written back as two bfloat16 numbers p = hi + lo (16 bits of mantissa);
//   4. O[64 x R] = O * corr + (P_hi + P_lo) V: warp w owns R / 8 columns of all 64 rows in registers.
// The learned sink enters the denominator at the end.  Tiles are found from cu_q on the device, so the launch
// depends on the step's shape alone.
#include "common.cuh"

namespace atom {

constexpr int kTcRows = 64;
constexpr int kTcKT = 32;
constexpr int kTcThreads = 256;
constexpr int kTcSStride = kTcKT + 1;      // floats
constexpr int kTcPStride = kTcKT + 8;      // bf16

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}

__device__ __forceinline__ void ldsm_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// NT: tiles of 8 value columns per warp; R = 64 * NT.
template <int NT>
__global__ void __launch_bounds__(kTcThreads, 1)
latent_attention_tc_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ q,
                           const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                           int page_size, const int* __restrict__ cu_q, const int* __restrict__ positions, int num_seqs,
                           int H, int HG, int TT, int rd, float scale, int window, const float* __restrict__ sink) {
  atom::pdl_trigger();
  constexpr int R = 64 * NT;
  const int Dk = R + rd, Dp = Dk + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [64][Dp]
  __nv_bfloat16* Ks = Qs + kTcRows * Dp;                                          // [2][32][Dp]
  __nv_bfloat16* Ph = Ks + 2 * kTcKT * Dp;                                        // [64][40]
  __nv_bfloat16* Pl = Ph + kTcRows * kTcPStride;                                  // [64][40]
  float* Ss = reinterpret_cast<float*>(Pl + kTcRows * kTcPStride);                // [64][33]
  float* ms = Ss + kTcRows * kTcSStride;                                          // [64]
  float* ls = ms + kTcRows;
  float* cs = ls + kTcRows;

  // which request and which of its tokens this CTA owns (read from the step's arrays: written before the step)
  int idx = blockIdx.x, s = 0, tok0 = -1, ntok = 0;
  for (; s < num_seqs; ++s) {
    const int a = cu_q[s], n = cu_q[s + 1] - a;
    const int tiles = (n + TT - 1) / TT;
    if (idx < tiles) {
      tok0 = a + idx * TT;
      ntok = min(TT, n - idx * TT);
      break;
    }
    idx -= tiles;
  }
  atom::pdl_wait();
  if (tok0 < 0) return;
  const int h0 = blockIdx.y * HG;
  const int hg = min(HG, H - h0);
  const int p0 = positions[tok0];
  const int k_lo = window > 0 ? max(0, p0 - window + 1) : 0;
  const int k_hi = p0 + ntok - 1;
  const int n_tiles = (k_hi - k_lo + kTcKT) / kTcKT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks_per_row = Dk / 8;

  auto load_tile = [&](int tile, int buf) {
    const int k0 = k_lo + tile * kTcKT;
    __nv_bfloat16* dst = Ks + buf * kTcKT * Dp;
    for (int c = tid; c < kTcKT * chunks_per_row; c += kTcThreads) {
      const int j = c / chunks_per_row, ch = c - j * chunks_per_row;
      const int key = k0 + j;
      if (key <= k_hi) {
        const int page = block_table[(int64_t)s * table_width + key / page_size];
        const __nv_bfloat16* src = pages + ((int64_t)page * page_size + key % page_size) * Dk + ch * 8;
        cp_async16(dst + j * Dp + ch * 8, src);
      } else {
        *reinterpret_cast<uint4*>(dst + j * Dp + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
  };

  load_tile(0, 0);
  // queries: 32-bit in, bfloat16 in shared memory; rows without a (token, head) are zeros
  for (int i = tid; i < kTcRows * Dk; i += kTcThreads) {
    const int r = i / Dk, d = i - r * Dk;
    const int ti = r / HG, hi = r - ti * HG;
    float v = 0.f;
    if (ti < ntok && hi < hg) v = q[((int64_t)(tok0 + ti) * H + h0 + hi) * Dk + d];
    Qs[r * Dp + d] = __float2bfloat16_rn(v);
  }
  for (int i = tid; i < kTcRows; i += kTcThreads) {
    ms[i] = -INFINITY;
    ls[i] = 0.f;
  }
  float acc[4][NT][4];
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mi][nt][e] = 0.f;

  const int g = lane >> 2, t4 = lane & 3;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    cp_async_wait_all();
    __syncthreads();                                    // tile's rows (and, the first time, Q) are in place
    if (tile + 1 < n_tiles) load_tile(tile + 1, buf ^ 1);
    const __nv_bfloat16* Kt = Ks + buf * kTcKT * Dp;
    const int k0 = k_lo + tile * kTcKT;
    {   // scores: this warp's 16 rows x 16 keys
      const int mi = warp >> 1, nb = (warp & 1) * 16;
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __nv_bfloat16* ap = Qs + (mi * 16 + (lane & 15)) * Dp + (lane >> 4) * 8;
      const __nv_bfloat16* bp = Kt + (nb + (lane & 7) + ((lane >> 4) << 3)) * Dp + ((lane >> 3) & 1) * 8;
      for (int kk = 0; kk < Dk; kk += 16) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldsm_x4(a0, a1, a2, a3, ap + kk);
        ldsm_x4(b0, b1, b2, b3, bp + kk);
        mma_bf16(sc[0], a0, a1, a2, a3, b0, b1);
        mma_bf16(sc[1], a0, a1, a2, a3, b2, b3);
      }
#pragma unroll
      for (int n2 = 0; n2 < 2; ++n2) {
        float* d0 = Ss + (mi * 16 + g) * kTcSStride + nb + n2 * 8 + 2 * t4;
        d0[0] = sc[n2][0];
        d0[1] = sc[n2][1];
        d0[8 * kTcSStride] = sc[n2][2];
        d0[8 * kTcSStride + 1] = sc[n2][3];
      }
    }
    __syncthreads();
    {   // softmax: warp w owns rows 8w .. 8w + 7, a lane is a key
      const int key = k0 + lane;
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        const int r = warp * 8 + rr;
        const int ti = r / HG;
        const int p = p0 + ti;
        const bool seen = ti < ntok && key <= p && key <= k_hi && (window <= 0 || p - key < window);
        const float sc = seen ? Ss[r * kTcSStride + lane] * scale : -INFINITY;
        const float m_old = ms[r];
        const float m_new = fmaxf(m_old, warp_max(sc));
        const float pw = (sc == -INFINITY) ? 0.f : expf(sc - m_new);
        const float sum = warp_sum(pw);
        const __nv_bfloat16 hi = __float2bfloat16_rn(pw);
        Ph[r * kTcPStride + lane] = hi;
        Pl[r * kTcPStride + lane] = __float2bfloat16_rn(pw - __bfloat162float(hi));
        __syncwarp();
        if (lane == 0) {
          const float corr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
          cs[r] = (m_new == -INFINITY) ? 1.f : corr;
          ms[r] = m_new;
          ls[r] = ls[r] * corr + sum;
        }
      }
    }
    __syncthreads();
    {   // output: this warp's R / 8 columns of all 64 rows
      float c[4][2];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi) {
        c[mi][0] = cs[mi * 16 + g];
        c[mi][1] = cs[mi * 16 + g + 8];
      }
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc[mi][nt][0] *= c[mi][0];
          acc[mi][nt][1] *= c[mi][0];
          acc[mi][nt][2] *= c[mi][1];
          acc[mi][nt][3] *= c[mi][1];
        }
      const int colbase = warp * 8 * NT;
#pragma unroll
      for (int ks = 0; ks < kTcKT / 16; ++ks) {
        uint32_t ah[4][4], al[4][4];
#pragma unroll
        for (int mi = 0; mi < 4; ++mi) {
          const int off = (mi * 16 + (lane & 15)) * kTcPStride + ks * 16 + (lane >> 4) * 8;
          ldsm_x4(ah[mi][0], ah[mi][1], ah[mi][2], ah[mi][3], Ph + off);
          ldsm_x4(al[mi][0], al[mi][1], al[mi][2], al[mi][3], Pl + off);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b0, b1;
          ldsm_x2_trans(b0, b1, Kt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * Dp + colbase + nt * 8);
#pragma unroll
          for (int mi = 0; mi < 4; ++mi) {
            mma_bf16(acc[mi][nt], ah[mi][0], ah[mi][1], ah[mi][2], ah[mi][3], b0, b1);
            mma_bf16(acc[mi][nt], al[mi][0], al[mi][1], al[mi][2], al[mi][3], b0, b1);
          }
        }
      }
    }
  }
  __syncthreads();
  // the sink joins the denominator; rows that are a (token, head) go out
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mi * 16 + g + half * 8;
      const int ti = r / HG, hi = r - ti * HG;
      if (ti >= ntok || hi >= hg) continue;
      const float m = ms[r], sk = sink ? sink[h0 + hi] : -INFINITY;
      const float top = fmaxf(m, sk);
      const float w = expf(m - top);
      const float inv = w / (ls[r] * w + (sink ? expf(sk - top) : 0.f));
      __nv_bfloat16* dst = out + ((int64_t)(tok0 + ti) * H + h0 + hi) * R + warp * 8 * NT + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(acc[mi][nt][half * 2] * inv, acc[mi][nt][half * 2 + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) = v;
      }
    }
}

static inline size_t latent_tc_smem(int R, int rd) {
  const int Dp = R + rd + 8;
  return sizeof(__nv_bfloat16) * ((size_t)kTcRows * Dp + 2 * (size_t)kTcKT * Dp + 2 * (size_t)kTcRows * kTcPStride) +
         sizeof(float) * ((size_t)kTcRows * kTcSStride + 3 * kTcRows);
}

template <int NT>
static int launch_latent_tc(__nv_bfloat16* out, const float* q, const __nv_bfloat16* pages, const int* block_table,
                            int table_width, int page_size, const int* cu_q, const int* positions, int num_seqs, int T,
                            int H, int rd, float scale, int window, const float* sink, cudaStream_t stream) {
  const int HG = H < kTcRows ? H : kTcRows;
  const int TT = kTcRows / HG;
  const size_t smem = latent_tc_smem(64 * NT, rd);
  auto k = latent_attention_tc_kernel<NT>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ATOM_ERR_LAUNCH;
  const dim3 grid((T + TT - 1) / TT + num_seqs, (H + HG - 1) / HG);
  launch_pdl(k, grid, dim3(kTcThreads), smem, stream, out, q, pages, block_table, table_width, page_size, cu_q, positions,
             num_seqs, H, HG, TT, rd, scale, window, sink);
  return check_launch();
}

}  // namespace atom

ATOM_EXPORT int atom_latent_attention_tc_supports(int H, int R, int rd) {
  if (H <= 0 || rd < 0 || rd % 16) return 0;
  if (R != 64 && R != 128 && R != 256 && R != 512) return 0;
  return atom::latent_tc_smem(R, rd) <= 220 * 1024;
}

// out: [T, H, R] bfloat16; q: [T, H, R + rd] float; pages: [pages, page, R + rd] bfloat16.
ATOM_EXPORT int atom_latent_attention_tc(void* out, const float* q, const void* pages, const int* block_table,
                                         int table_width, int page_size, const int* cu_q, const int* positions,
                                         int num_seqs, int T, int H, int R, int rd, float scale, int window,
                                         const float* sink, cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (!atom_latent_attention_tc_supports(H, R, rd) || page_size <= 0 || window < 0) return ATOM_ERR_ARG;
  auto* o = (__nv_bfloat16*)out;
  auto* pg = (const __nv_bfloat16*)pages;
  switch (R) {
    case 64: return atom::launch_latent_tc<1>(o, q, pg, block_table, table_width, page_size, cu_q, positions, num_seqs, T, H, rd, scale, window, sink, stream);
    case 128: return atom::launch_latent_tc<2>(o, q, pg, block_table, table_width, page_size, cu_q, positions, num_seqs, T, H, rd, scale, window, sink, stream);
    case 256: return atom::launch_latent_tc<4>(o, q, pg, block_table, table_width, page_size, cu_q, positions, num_seqs, T, H, rd, scale, window, sink, stream);
    case 512: return atom::launch_latent_tc<8>(o, q, pg, block_table, table_width, page_size, cu_q, positions, num_seqs, T, H, rd, scale, window, sink, stream);
  }
  return ATOM_ERR_ARG;
}
