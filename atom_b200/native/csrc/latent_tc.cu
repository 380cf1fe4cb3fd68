// Attention over a cached latent on the tensor cores (bfloat16; see latent.cu for the mechanism and the plain
// kernel).  Because every head reads the same row [c | kr] per key, the heads of a token are rows of one
// product: a CTA owns 64 query rows = a few consecutive tokens of one request x a group of heads (16 rows in
// steps of single tokens), and walks the keys its tokens may see, or its share of them, in tiles of 32:
//   1. the tile's rows come into shared memory once (cp.async, two buffers): they are the K operand of the
//      scores AND, in their first R columns, the V operand of the output;
//   2. S[64 x 32] = Q K^T on mma.sync m16n8k16 (each warp two 16 x 8 tiles over all R + rd columns), 32-bit sums;
//   3. scale, window and causal mask, running maximum and sum per row in 32-bit.  64-row tiles do this on the
//      score fragments (a row's statistics through the quads and one exchange between the two warps that hold the
//      row); 16-row tiles add the warps' partial scores in shared memory, a warp per two rows and a lane per key.
//      The weights go to shared memory as two bfloat16 numbers p = hi + lo (16 bits of mantissa);
//   4. O[64 x R] = O * corr + (P_hi + P_lo) V: warp w owns R / 8 columns of all 64 rows in registers.
// The learned sink enters the denominator at the end, or in the merge kernel when the keys were shared out.
// Tiles are found from cu_q on the device, so the launch depends on the step's shape alone.
#include "common.cuh"

namespace atom {

constexpr int kTcKT = 32;
constexpr int kTcThreads = 256;
static_assert(kTcThreads == 8 * kTcKT, "eight threads copy a key row");
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

// NT: tiles of 8 value columns per warp; R = 64 * NT.  MI: tiles of 16 query rows per CTA, 4 for steps with prompt
// portions; 1 for steps of single tokens, where a CTA's rows are one token's heads: the warps then share out the
// columns of Q and K of one row tile (kTcSlices partial scores that the softmax adds), and two CTAs fit an SM.
template <int NT, int MI>
__global__ void __launch_bounds__(kTcThreads, MI == 1 ? 2 : 1)
latent_attention_tc_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ q,
                           const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                           int page_size, const int* __restrict__ cu_q, const int* __restrict__ positions, int num_seqs,
                           int H, int HG, int TT, int rd, float scale, int window, const float* __restrict__ sink,
                           float* __restrict__ scratch, int nsplit) {
  atom::pdl_trigger();
  constexpr int R = 64 * NT;
  constexpr int kTcRows = 16 * MI;
  constexpr int kSlices = MI == 1 ? 4 : 1;
  const int Dk = R + rd, Dp = Dk + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [64][Dp]
  __nv_bfloat16* Ks = Qs + kTcRows * Dp;                                          // [2][32][Dp]
  __nv_bfloat16* Ph = Ks + 2 * kTcKT * Dp;                                        // [64][40]
  __nv_bfloat16* Pl = Ph + kTcRows * kTcPStride;                                  // [64][40]
  float* Ss = reinterpret_cast<float*>(Pl + kTcRows * kTcPStride);                // [slices][rows][33]
  float* ms = Ss + kSlices * kTcRows * kTcSStride;                                // [rows]
  float* ls = ms + kTcRows;
  float* cs = ls + kTcRows;
  // MI == 4 keeps its scores in registers; where they would lie are two halves' row maxima and sums, and the running
  // maximum twice (read from one, written to the other, so that both warps of a row read the same old value)
  float* pm = Ss;                      // [rows][2]
  float* psum = pm + 2 * kTcRows;      // [rows][2]
  if (MI == 4) ms = psum + 2 * kTcRows;     // [2][rows]
  int par = 0;

  // which request and which of its tokens this CTA owns (read from the step's arrays: written before the step)
  int idx = blockIdx.x, s = 0, tok0 = -1, ntok = 0;
  for (; s < num_seqs; ++s) {
    const int a = cu_q[s], n = cu_q[s + 1] - a;
    const int tiles = (n + TT - 1) / TT;
    if (idx < tiles) {
      idx = tiles - 1 - idx;      // a request's last tiles see the most keys: they start first
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
  // with nsplit > 1 this CTA walks one share of the tiles and leaves unnormalised sums for the merge kernel
  int tile_begin = 0, tile_end = n_tiles;
  if (nsplit > 1) {
    const int per = (n_tiles + nsplit - 1) / nsplit;
    tile_begin = min(n_tiles, (int)blockIdx.z * per);
    tile_end = min(n_tiles, tile_begin + per);
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks_per_row = Dk / 8;

  // a tile's row j is copied by threads 8 j .. 8 j + 7 in chunks of 16 bytes: one page lookup per thread and tile
  const int lrow = tid >> 3, lch = tid & 7;
  auto load_tile = [&](int tile, int buf) {
    const int key = k_lo + tile * kTcKT + lrow;
    __nv_bfloat16* dst = Ks + (buf * kTcKT + lrow) * Dp;
    if (key <= k_hi) {
      const int pg = key / page_size;
      const int page = block_table[(int64_t)s * table_width + pg];
      const __nv_bfloat16* src = pages + ((int64_t)page * page_size + (key - pg * page_size)) * Dk;
      for (int ch = lch; ch < chunks_per_row; ch += 8) cp_async16(dst + ch * 8, src + ch * 8);
    } else {
      for (int ch = lch; ch < chunks_per_row; ch += 8) *reinterpret_cast<uint4*>(dst + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    cp_async_commit();
  };

  if (tile_begin < tile_end) load_tile(tile_begin, 0);
  // queries: 32-bit in, bfloat16 in shared memory; rows without a (token, head) are zeros
  const int q4 = Dk / 4;
  for (int i = tid; i < kTcRows * q4; i += kTcThreads) {
    const int r = i / q4, d = (i - r * q4) * 4;
    const int ti = r / HG, hi = r - ti * HG;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ti < ntok && hi < hg) v = *reinterpret_cast<const float4*>(q + ((int64_t)(tok0 + ti) * H + h0 + hi) * Dk + d);
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(Qs + r * Dp + d);
    dst[0] = __floats2bfloat162_rn(v.x, v.y);
    dst[1] = __floats2bfloat162_rn(v.z, v.w);
  }
  for (int i = tid; i < kTcRows; i += kTcThreads) {
    ms[i] = -INFINITY;
    if (MI == 4) ms[kTcRows + i] = -INFINITY;
    ls[i] = 0.f;
  }
  float acc[MI][NT][4];
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mi][nt][e] = 0.f;

  const int g = lane >> 2, t4 = lane & 3;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int buf = (tile - tile_begin) & 1;
    cp_async_wait_all();
    __syncthreads();                                    // tile's rows (and, the first time, Q) are in place
    if (tile + 1 < tile_end) load_tile(tile + 1, buf ^ 1);
    const __nv_bfloat16* Kt = Ks + buf * kTcKT * Dp;
    const int k0 = k_lo + tile * kTcKT;
    {   // scores: this warp's 16 rows x 16 keys (over its slice of the columns)
      const int mi = MI == 1 ? 0 : warp >> 1, nb = (warp & 1) * 16;
      const int slice = MI == 1 ? warp >> 1 : 0;
      const int steps = Dk / 16, per_slice = (steps + kSlices - 1) / kSlices;
      const int k_end = min(steps, (slice + 1) * per_slice) * 16;
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float sd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};     // odd steps: four sums in flight, not two
      const __nv_bfloat16* ap = Qs + (mi * 16 + (lane & 15)) * Dp + (lane >> 4) * 8;
      const __nv_bfloat16* bp = Kt + (nb + (lane & 7) + ((lane >> 4) << 3)) * Dp + ((lane >> 3) & 1) * 8;
      int kk = slice * per_slice * 16;
      for (; kk + 32 <= k_end; kk += 32) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, d0, d1, d2, d3;
        ldsm_x4(a0, a1, a2, a3, ap + kk);
        ldsm_x4(b0, b1, b2, b3, bp + kk);
        ldsm_x4(c0, c1, c2, c3, ap + kk + 16);
        ldsm_x4(d0, d1, d2, d3, bp + kk + 16);
        mma_bf16(sc[0], a0, a1, a2, a3, b0, b1);
        mma_bf16(sc[1], a0, a1, a2, a3, b2, b3);
        mma_bf16(sd[0], c0, c1, c2, c3, d0, d1);
        mma_bf16(sd[1], c0, c1, c2, c3, d2, d3);
      }
      if (kk < k_end) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldsm_x4(a0, a1, a2, a3, ap + kk);
        ldsm_x4(b0, b1, b2, b3, bp + kk);
        mma_bf16(sc[0], a0, a1, a2, a3, b0, b1);
        mma_bf16(sc[1], a0, a1, a2, a3, b2, b3);
      }
#pragma unroll
      for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[n2][e] += sd[n2][e];
      if constexpr (MI == 4) {
        // softmax on the fragments: a thread holds rows g and g + 8 of its warp's tile at keys nb + 8 n2 + 2 t4 + e;
        // the row's other keys are in its three neighbours of the quad and in the warp beside this one
        const int half_of_row = warp & 1;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = mi * 16 + g + 8 * hf;
          const int ti = r / HG;
          const int p = p0 + ti;
#pragma unroll
          for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int key = k0 + nb + n2 * 8 + 2 * t4 + e;
              const bool seen = ti < ntok && key <= p && key <= k_hi && (window <= 0 || p - key < window);
              const float v = seen ? sc[n2][2 * hf + e] * scale : -INFINITY;
              sc[n2][2 * hf + e] = v;
              mx[hf] = fmaxf(mx[hf], v);
            }
          mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
          mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
          if (t4 == 0) pm[r * 2 + half_of_row] = mx[hf];
        }
        __syncthreads();
        const float* m_cur = ms + par * kTcRows;
        float* m_nxt = ms + (par ^ 1) * kTcRows;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = mi * 16 + g + 8 * hf;
          const float m_old = m_cur[r];
          const float m_new = fmaxf(m_old, fmaxf(pm[r * 2], pm[r * 2 + 1]));
          float sum = 0.f;
#pragma unroll
          for (int n2 = 0; n2 < 2; ++n2) {
            const float w0 = sc[n2][2 * hf] == -INFINITY ? 0.f : expf(sc[n2][2 * hf] - m_new);
            const float w1 = sc[n2][2 * hf + 1] == -INFINITY ? 0.f : expf(sc[n2][2 * hf + 1] - m_new);
            sum += w0 + w1;
            const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(w0 - __low2float(hi), w1 - __high2float(hi));
            const int at = r * kTcPStride + nb + n2 * 8 + 2 * t4;
            *reinterpret_cast<__nv_bfloat162*>(Ph + at) = hi;
            *reinterpret_cast<__nv_bfloat162*>(Pl + at) = lo;
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          if (t4 == 0) {
            psum[r * 2 + half_of_row] = sum;
            if (half_of_row == 0) {
              const float corr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
              cs[r] = (m_new == -INFINITY) ? 1.f : corr;
              m_nxt[r] = m_new;
            }
          }
        }
      } else {
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {
          float* d0 = Ss + (slice * kTcRows + mi * 16 + g) * kTcSStride + nb + n2 * 8 + 2 * t4;
          d0[0] = sc[n2][0];
          d0[1] = sc[n2][1];
          d0[8 * kTcSStride] = sc[n2][2];
          d0[8 * kTcSStride + 1] = sc[n2][3];
        }
        __syncthreads();
        // softmax: warp w owns rows 2 w and 2 w + 1, a lane is a key; the slices' partial scores are added here
        const int key = k0 + lane;
#pragma unroll
        for (int rr = 0; rr < 2 * MI; ++rr) {
          const int r = warp * 2 * MI + rr;
          const int ti = r / HG;
          const int p = p0 + ti;
          const bool seen = ti < ntok && key <= p && key <= k_hi && (window <= 0 || p - key < window);
          float raw = Ss[r * kTcSStride + lane];
#pragma unroll
          for (int sl = 1; sl < kSlices; ++sl) raw += Ss[(sl * kTcRows + r) * kTcSStride + lane];
          const float sv = seen ? raw * scale : -INFINITY;
          const float m_old = ms[r];
          const float m_new = fmaxf(m_old, warp_max(sv));
          const float pw = (sv == -INFINITY) ? 0.f : expf(sv - m_new);
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
    }
    __syncthreads();
    {   // output: this warp's R / 8 columns of all rows
      if (MI == 4) {
        par ^= 1;
        if (tid < kTcRows) ls[tid] = ls[tid] * cs[tid] + psum[2 * tid] + psum[2 * tid + 1];
      }
      float c[MI][2];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi) {
        c[mi][0] = cs[mi * 16 + g];
        c[mi][1] = cs[mi * 16 + g + 8];
      }
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
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
        uint32_t ah[MI][4], al[MI][4];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          const int off = (mi * 16 + (lane & 15)) * kTcPStride + ks * 16 + (lane >> 4) * 8;
          ldsm_x4(ah[mi][0], ah[mi][1], ah[mi][2], ah[mi][3], Ph + off);
          ldsm_x4(al[mi][0], al[mi][1], al[mi][2], al[mi][3], Pl + off);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b0, b1;
          ldsm_x2_trans(b0, b1, Kt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * Dp + colbase + nt * 8);
#pragma unroll
          for (int mi = 0; mi < MI; ++mi) {
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
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mi * 16 + g + half * 8;
      const int ti = r / HG, hi = r - ti * HG;
      if (ti >= ntok || hi >= hg) continue;
      if (nsplit > 1) {
        float* dst = scratch + (((int64_t)(tok0 + ti) * H + h0 + hi) * nsplit + blockIdx.z) * (R + 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          *reinterpret_cast<float2*>(dst + warp * 8 * NT + nt * 8 + 2 * t4) =
              make_float2(acc[mi][nt][half * 2], acc[mi][nt][half * 2 + 1]);
        if (warp == 0 && t4 == 0) {
          dst[R] = ms[par * kTcRows + r];
          dst[R + 1] = ls[r];
        }
        continue;
      }
      const float m = ms[par * kTcRows + r], sk = sink ? sink[h0 + hi] : -INFINITY;
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

static inline size_t latent_tc_smem(int R, int rd, int rows) {
  const int Dp = R + rd + 8, slices = rows == 16 ? 4 : 1;
  return sizeof(__nv_bfloat16) * ((size_t)rows * Dp + 2 * (size_t)kTcKT * Dp + 2 * (size_t)rows * kTcPStride) +
         sizeof(float) * ((size_t)slices * rows * kTcSStride + 3 * rows);
}

template <int NT, int MI>
static int launch_latent_tc(__nv_bfloat16* out, const float* q, const __nv_bfloat16* pages, const int* block_table,
                            int table_width, int page_size, const int* cu_q, const int* positions, int num_seqs, int T,
                            int H, int rd, float scale, int window, const float* sink, float* scratch, int nsplit,
                            cudaStream_t stream) {
  constexpr int kTcRows = 16 * MI;
  const int HG = H < kTcRows ? H : kTcRows;
  const int TT = kTcRows / HG;
  const size_t smem = latent_tc_smem(64 * NT, rd, kTcRows);
  auto k = latent_attention_tc_kernel<NT, MI>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ATOM_ERR_LAUNCH;
  const dim3 grid((T + TT - 1) / TT + num_seqs, (H + HG - 1) / HG, nsplit);
  launch_pdl(k, grid, dim3(kTcThreads), smem, stream, out, q, pages, block_table, table_width, page_size, cu_q, positions,
             num_seqs, H, HG, TT, rd, scale, window, sink, scratch, nsplit);
  return check_launch();
}

}  // namespace atom

ATOM_EXPORT int atom_latent_attention_tc_supports(int H, int R, int rd) {
  if (H <= 0 || rd < 0 || rd % 16) return 0;
  if (R < 64 || R > 512 || R % 64) return 0;
  return atom::latent_tc_smem(R, rd, 64) <= 220 * 1024;
}

// out: [T, H, R] bfloat16; q: [T, H, R + rd] float; pages: [pages, page, R + rd] bfloat16.  rows: 64 query rows per
// CTA (steps with prompt portions) or 16 (steps of single tokens).  nsplit > 1: partial sums to scratch
// [T, H, nsplit, R + 2], to be put together by atom_latent_merge.
ATOM_EXPORT int atom_latent_attention_tc(void* out, const float* q, const void* pages, const int* block_table,
                                         int table_width, int page_size, const int* cu_q, const int* positions,
                                         int num_seqs, int T, int H, int R, int rd, float scale, int window,
                                         const float* sink, float* scratch, int nsplit, int rows, cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (!atom_latent_attention_tc_supports(H, R, rd) || page_size <= 0 || window < 0 || nsplit < 1 || nsplit > 65535 ||
      (nsplit > 1 && !scratch) || (rows != 16 && rows != 64))
    return ATOM_ERR_ARG;
  auto* o = (__nv_bfloat16*)out;
  auto* pg = (const __nv_bfloat16*)pages;
#define ATOM_LATENT_TC(NT)                                                                                            \
  return rows == 16 ? atom::launch_latent_tc<NT, 1>(o, q, pg, block_table, table_width, page_size, cu_q, positions,   \
                                                    num_seqs, T, H, rd, scale, window, sink, scratch, nsplit, stream) \
                    : atom::launch_latent_tc<NT, 4>(o, q, pg, block_table, table_width, page_size, cu_q, positions,   \
                                                    num_seqs, T, H, rd, scale, window, sink, scratch, nsplit, stream)
  switch (R) {
    case 64: ATOM_LATENT_TC(1);
    case 128: ATOM_LATENT_TC(2);
    case 192: ATOM_LATENT_TC(3);
    case 256: ATOM_LATENT_TC(4);
    case 320: ATOM_LATENT_TC(5);
    case 384: ATOM_LATENT_TC(6);
    case 448: ATOM_LATENT_TC(7);
    case 512: ATOM_LATENT_TC(8);
  }
#undef ATOM_LATENT_TC
  return ATOM_ERR_ARG;
}
