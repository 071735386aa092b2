// Attention over a cached latent on the tensor cores, for bfloat16 pages: what
// asb_latent_attention (latent_attention.cu, the float32 path and the fallback) computes, with
// Q K^T and P V as mma.sync m16n8k16 (bfloat16 in, float32 accumulate).
//
// A block owns 32 (token, head) rows, the heads of one or a few neighbouring tokens of a
// request, which all read the same keys: one shared key head of width Dk = rank + rot, whose
// first `rank` entries are also the values. Per tile of 64 keys, staged once in shared memory
// (cp.async, the next tile arriving while this one is multiplied):
//   1. each of the 8 warps multiplies the 32 query rows with 8 of the keys (k over Dk) and
//      writes the scaled, masked float32 scores to shared memory;
//   2. each warp runs the online softmax of 4 of the rows: running maximum and sum in float32,
//      the weights written as bfloat16, the factor by which older sums shrink kept per row;
//   3. each warp multiplies the 32 x 64 weights with the keys' first `rank` columns for its own
//      eighth of the output columns (the keys read through ldmatrix.trans as the B operand).
// Scores, maxima, sums and the output accumulators are float32; the queries and the softmax
// weights enter the tensor cores rounded to bfloat16. Key partitions, their alignment to
// absolute positions and the partial results are those of the CUDA-core kernel, merged by
// asb_attention_reduce.
#include "common.cuh"

namespace {

constexpr int MR = 32;   // rows a block
constexpr int KT = 64;   // keys a tile
constexpr int kWarps = 8;
constexpr int LDS = KT + 1;  // float32 scores
constexpr int LDP = KT + 8;  // bfloat16 weights

struct LatentParams {
  const float* q;            // [T, H, Dk]
  float* out;                // [T, H, rank]
  const __nv_bfloat16* pages;  // [num_blocks, 1, bs, Dk]
  const int* block_tables;
  const int* req_q_start;
  const int* req_pos_start;
  float* part_m;
  float* part_l;
  float* part_acc;
  int R, H, rank, Dk, DKP, LDK, bs, table_width;
  int QT, GC, HC;
  int PS, NP;
  float scale;
  int window;  // > 0: a query at p sees keys j with p - j < window only
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&b)[2], const void* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// NT: 8-column tiles of the output per warp; the block covers 64 * NT >= rank columns
template <int NT>
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_mma_kernel(const LatentParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Dk = p.Dk, Dv = p.rank, DKP = p.DKP, LDK = p.LDK;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [MR][LDK]
  __nv_bfloat16* k_buf = q_s + MR * LDK;                             // 2 x [KT][LDK]: one tile multiplied, the next one arriving
  __nv_bfloat16* p_s = k_buf + 2 * KT * LDK;                         // [MR][LDP]
  float* s_s = reinterpret_cast<float*>(p_s + MR * LDP);             // [MR][LDS]
  float* row_m = s_s + MR * LDS;                                     // [MR]
  float* row_l = row_m + MR;
  float* row_c = row_l + MR;
  __shared__ int block_of_key[KT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  int tile = blockIdx.x, r = 0, q_len = 0;
  for (; r < p.R; ++r) {
    q_len = p.req_q_start[r + 1] - p.req_q_start[r];
    const int tiles = (q_len + p.QT - 1) / p.QT;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (r == p.R) return;
  const int q0 = tile * p.QT;
  const int nq = min(p.QT, q_len - q0);
  const int row0 = p.req_q_start[r] + q0;
  const int pos0 = p.req_pos_start[r] + q0;
  const int head0 = blockIdx.y * p.GC;
  const int gc = min(p.GC, p.H - head0);
  const int num_rows = nq * gc;  // row rr = qi * gc + g
  const int hi = pos0 + nq;
  // with a window no row of the tile sees a key before pos0 - window + 1 (pages before it may be gone)
  const int key_lo = max((int)blockIdx.z * p.PS, p.window > 0 ? pos0 - p.window + 1 : 0);
  const int key_hi = (int)min((long long)hi, (long long)(blockIdx.z + 1) * p.PS);

  // queries as bfloat16, a warp per row, rows beyond the block's and columns beyond Dk zero
  const bool q4 = (Dk % 4 == 0) && (((uintptr_t)p.q & 15) == 0);
  for (int rr = warp; rr < MR; rr += kWarps) {
    __nv_bfloat16* dst = q_s + rr * LDK;
    const float* src = nullptr;
    if (rr < num_rows) {
      const int qi = rr / gc, gg = rr - qi * gc;
      src = p.q + ((size_t)(row0 + qi) * p.H + head0 + gg) * Dk;
    }
    if (src && q4) {
      for (int e = lane * 4; e < Dk; e += 128) {
        const float4 v = *reinterpret_cast<const float4*>(src + e);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + e) = packed;
      }
      for (int e = Dk + lane; e < LDK; e += 32) dst[e] = __float2bfloat16_rn(0.f);
    } else {
      for (int e = lane; e < LDK; e += 32) dst[e] = __float2bfloat16_rn((src && e < Dk) ? src[e] : 0.f);
    }
  }
  // the key tiles' columns beyond Dk stay zero (every tile rewrites the Dk columns of all its rows)
  for (int i = threadIdx.x; i < 2 * KT * (LDK - Dk); i += blockDim.x) {
    const int jj = i / (LDK - Dk), e = Dk + i - jj * (LDK - Dk);
    k_buf[jj * LDK + e] = __float2bfloat16_rn(0.f);
  }
  if (threadIdx.x < MR) {
    row_m[threadIdx.x] = -INFINITY;
    row_l[threadIdx.x] = 0.f;
  }
  float acc[2][NT][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  // the positions of the four rows whose scores this thread writes, once (a division each)
  int row_pos[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int rr = i * 16 + g + half * 8;
      row_pos[i][half] = rr < num_rows ? pos0 + rr / gc : -1;
    }
  const int* table = p.block_tables + (size_t)r * p.table_width;
  const bool vector = (Dk % 8 == 0) && (((uintptr_t)p.pages & 15) == 0);
  const int chunks = Dk / 8;

  // A tile's keys: 16-byte asynchronous copies where the rows allow them (Dk a multiple of 8),
  // keys outside the block's range filled with zeros; the tile after the one being multiplied is
  // always on its way. Other widths are copied element by element when their turn comes.
  auto request_tile = [&](int kt0, __nv_bfloat16* k_s) {
    // a warp fetches 8 of the tile's keys: lanes 0-7 look up where they lie (one division each a
    // tile), then all lanes copy each key's chunks
    const int jw = kt0 + warp * 8 + (lane & 7);
    long long mine = -1;
    if (jw >= key_lo && jw < key_hi) mine = (long long)table[jw / p.bs] * p.bs + jw % p.bs;
#pragma unroll
    for (int r8 = 0; r8 < 8; ++r8) {
      const long long slot = __shfl_sync(0xffffffffu, mine, r8);
      const __nv_bfloat16* src = slot >= 0 ? p.pages + (size_t)slot * Dk : p.pages;
      __nv_bfloat16* dst = k_s + (warp * 8 + r8) * LDK;
      for (int c = lane; c < chunks; c += 32) {
        const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + c * 8);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(slot >= 0 ? src + c * 8 : src), "r"(slot >= 0 ? 16 : 0) : "memory");
      }
    }
  };
  const int first_tile = (key_lo / KT) * KT;
  __syncthreads();  // the zeros are in place before any copy lands on them
  if (vector && first_tile < key_hi) request_tile(first_tile, k_buf);
  asm volatile("cp.async.commit_group;" ::: "memory");

  for (int kt0 = first_tile, turn = 0; kt0 < key_hi; kt0 += KT, turn ^= 1) {
    __nv_bfloat16* k_s = k_buf + turn * KT * LDK;
    if (threadIdx.x < KT) {
      const int j = kt0 + threadIdx.x;
      block_of_key[threadIdx.x] = (j >= key_lo && j < key_hi) ? table[j / p.bs] : -1;
    }
    if (vector) {
      if (kt0 + KT < key_hi) request_tile(kt0 + KT, k_buf + (turn ^ 1) * KT * LDK);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest group: this tile has arrived
    } else {
      __syncthreads();
      for (int i = threadIdx.x; i < KT * Dk; i += blockDim.x) {
        const int jj = i / Dk, e = i - jj * Dk;
        const int blk = block_of_key[jj];
        k_s[jj * LDK + e] = blk >= 0 ? p.pages[((size_t)blk * p.bs + (kt0 + jj) % p.bs) * Dk + e] : __float2bfloat16_rn(0.f);
      }
    }
    __syncthreads();

    // 1. scores of the 32 rows against this warp's 8 keys
    {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      // fragments by ldmatrix: a lane names one row of one 8 x 8 block. Queries: rows (lane % 16) of
      // each 16-row tile, k block lane / 16; keys: this warp's 8 keys, k block (lane / 8) % 2 (x2) or
      // lane / 8 (x4, two k steps at once)
      const __nv_bfloat16* qa0 = q_s + (lane & 15) * LDK + (lane >> 4) * 8;
      const __nv_bfloat16* qa1 = qa0 + 16 * LDK;
      const __nv_bfloat16* kb = k_s + (warp * 8 + (lane & 7)) * LDK + (lane >> 3) * 8;
      int kk = 0;
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // odd k steps: four chains of dependent MMAs, not two
#pragma unroll 2
      for (; kk + 32 <= DKP; kk += 32) {
        uint32_t b4[4], a0[4], a1[4], a2[4], a3[4];
        ldmatrix_x4(b4, kb + kk);
        ldmatrix_x4(a0, qa0 + kk);
        ldmatrix_x4(a1, qa1 + kk);
        ldmatrix_x4(a2, qa0 + kk + 16);
        ldmatrix_x4(a3, qa1 + kk + 16);
        const uint32_t b_lo[2] = {b4[0], b4[1]}, b_hi[2] = {b4[2], b4[3]};
        mma_bf16(s[0], a0, b_lo);
        mma_bf16(s[1], a1, b_lo);
        mma_bf16(s2[0], a2, b_hi);
        mma_bf16(s2[1], a3, b_hi);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[i][c] += s2[i][c];
      if (kk < DKP) {
        uint32_t b[2], a[4];
        ldmatrix_x2(b, k_s + (warp * 8 + (lane & 7)) * LDK + ((lane >> 3) & 1) * 8 + kk);
        ldmatrix_x4(a, qa0 + kk);
        mma_bf16(s[0], a, b);
        ldmatrix_x4(a, qa1 + kk);
        mma_bf16(s[1], a, b);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int rr = i * 16 + g + (c >> 1) * 8;
          const int jj = warp * 8 + 2 * t + (c & 1);
          const int j = kt0 + jj;
          const bool visible = j >= key_lo && j < key_hi && j <= row_pos[i][c >> 1] && (p.window <= 0 || row_pos[i][c >> 1] - j < p.window);  // (no position for rows beyond the block's)
          s_s[rr * LDS + jj] = visible ? s[i][c] * p.scale : -INFINITY;
        }
    }
    __syncthreads();

    // 2. online softmax, 4 rows a warp, two keys a lane
#pragma unroll
    for (int u = 0; u < MR / kWarps; ++u) {
      const int rr = warp * (MR / kWarps) + u;
      const float s0 = s_s[rr * LDS + lane], s1 = s_s[rr * LDS + lane + 32];
      const float m_old = row_m[rr];
      const float m_new = fmaxf(m_old, asb::warp_max(fmaxf(s0, s1)));
      float p0 = 0.f, p1 = 0.f, corr = 1.f;
      if (m_new != -INFINITY) {
        p0 = expf(s0 - m_new);
        p1 = expf(s1 - m_new);
        corr = expf(m_old - m_new);
      }
      const float sum = asb::warp_sum(p0 + p1);
      p_s[rr * LDP + lane] = __float2bfloat16_rn(p0);
      p_s[rr * LDP + lane + 32] = __float2bfloat16_rn(p1);
      if (lane == 0) {
        row_m[rr] = m_new;
        row_l[rr] = row_l[rr] * corr + sum;
        row_c[rr] = corr;
      }
    }
    __syncthreads();

    // 3. the weighted sum of the keys' value columns, this warp's columns
    {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float c_lo = row_c[i * 16 + g], c_hi = row_c[i * 16 + g + 8];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          acc[i][j][0] *= c_lo;
          acc[i][j][1] *= c_lo;
          acc[i][j][2] *= c_hi;
          acc[i][j][3] *= c_hi;
        }
      }
      const int col0 = warp * NT * 8;
#pragma unroll
      for (int kk = 0; kk < KT; kk += 16) {
        uint32_t a[2][4];
        ldmatrix_x4(a[0], p_s + (lane & 15) * LDP + kk + (lane >> 4) * 8);
        ldmatrix_x4(a[1], p_s + (16 + (lane & 15)) * LDP + kk + (lane >> 4) * 8);
        if constexpr (NT >= 2) {
          // two 8-column tiles per ldmatrix: keys kk + lane % 16, columns of tile j + lane / 16
#pragma unroll
          for (int j = 0; j < NT; j += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, k_s + (kk + (lane & 15)) * LDK + col0 + (j + (lane >> 4)) * 8);
            const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
            mma_bf16(acc[0][j], a[0], b0);
            mma_bf16(acc[1][j], a[1], b0);
            mma_bf16(acc[0][j + 1], a[0], b1);
            mma_bf16(acc[1][j + 1], a[1], b1);
          }
        } else {
          uint32_t b[2];
          ldmatrix_x2_trans(b, k_s + (kk + (lane & 15)) * LDK + col0);
          mma_bf16(acc[0][0], a[0], b);
          mma_bf16(acc[1][0], a[1], b);
        }
      }
    }
    __syncthreads();  // this tile's keys, weights and key table have been read
  }

#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int rr = i * 16 + g + half * 8;
      if (rr >= num_rows) continue;
      const int qi = rr / gc, gg = rr - qi * gc;
      const size_t row = (size_t)(row0 + qi) * p.H + head0 + gg;
      const float l = row_l[rr];
      if (p.NP > 1 && warp == 0 && t == 0) {
        p.part_m[row * p.NP + blockIdx.z] = row_m[rr];
        p.part_l[row * p.NP + blockIdx.z] = l;
      }
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = warp * NT * 8 + j * 8 + 2 * t + c;
          if (col >= Dv) continue;
          const float v = acc[i][j][half * 2 + c];
          if (p.NP == 1) p.out[row * Dv + col] = v / l;
          else p.part_acc[(row * p.NP + blockIdx.z) * Dv + col] = v;
        }
    }
}

// ---- per-head products on the tensor cores ------------------------------------------------------
//
// out[t, h, :] = x[t, h, :] . w[h]^T for w [H, N, K] (bfloat16, K contiguous), optionally times
// sigmoid(gate[t, h]): the query absorption (x bfloat16, out float32) and the value up-projection
// with the output gate (x float32, rounded to bfloat16 on the way in; out bfloat16). A block
// computes 64 tokens x 64 columns of one head, four warps of 32 x 32, K in steps of 32.

constexpr int HB = 64, HK = 32, HLD = HK + 8;

template <typename TX, typename TO>
__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(TO* __restrict__ out, int out_row, int out_head, const TX* __restrict__ x, int x_row, int x_head,
                       const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ gate, int gate_row,
                       int T, int K, int N) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  __shared__ __align__(16) __nv_bfloat16 xs[HB][HLD];
  __shared__ __align__(16) __nv_bfloat16 ws[HB][HLD];
  const int t0 = blockIdx.x * HB, h = blockIdx.y, n0 = blockIdx.z * HB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  const int lrow0 = tid >> 2, lrow1 = lrow0 + 32, lchunk = (tid & 3) * 8;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HK) {
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int lr = half ? lrow1 : lrow0;
      const int tok = t0 + lr, n = n0 + lr, k = k0 + lchunk;
      uint4 wv = make_uint4(0, 0, 0, 0);
      if (n < N && k < K) wv = *reinterpret_cast<const uint4*>(wh + (size_t)n * K + k);
      *reinterpret_cast<uint4*>(&ws[lr][lchunk]) = wv;
      const TX* xp = x + (size_t)tok * x_row + (size_t)h * x_head + k;
#pragma unroll
      for (int u = 0; u < 8; ++u) xs[lr][lchunk + u] = (tok < T && k + u < K) ? __float2bfloat16_rn(asb::to_float(xp[u])) : __float2bfloat16_rn(0.f);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + g;
        a[i][0] = *reinterpret_cast<const uint32_t*>(&xs[r][kk + 2 * t]);
        a[i][1] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kk + 2 * t]);
        a[i][2] = *reinterpret_cast<const uint32_t*>(&xs[r][kk + 2 * t + 8]);
        a[i][3] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + j * 8 + g;
        uint32_t b[2];
        b[0] = *reinterpret_cast<const uint32_t*>(&ws[n][kk + 2 * t]);
        b[1] = *reinterpret_cast<const uint32_t*>(&ws[n][kk + 2 * t + 8]);
        mma_bf16(acc[0][j], a[0], b);
        mma_bf16(acc[1][j], a[1], b);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int tok = t0 + wm + i * 16 + g + half * 8;
      if (tok >= T) continue;
      float scale = 1.f;
      if (gate) scale = 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)tok * gate_row + h])));
      TO* orow = out + (size_t)tok * out_row + (size_t)h * out_head;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn + j * 8 + 2 * t + c;
          if (n < N) orow[n] = asb::from_float<TO>(acc[i][j][half * 2 + c] * scale);
        }
    }
}

}  // namespace

extern "C" int asb_head_matmul_mma_supported(int K) { return K >= 8 && K % 8 == 0; }

// w: [H, N, K] bfloat16. x: float32 (x_f32 1) or bfloat16; out: float32 (out_f32 1) or bfloat16.
extern "C" int asb_head_matmul_mma(void* out, int out_f32, int out_row, int out_head, const void* x, int x_f32, int x_row,
                                   int x_head, const void* w, const void* gate, int gate_row, int T, int H, int K, int N,
                                   cudaStream_t stream) {
  if (T == 0) return 0;
  if (!asb_head_matmul_mma_supported(K) || ((uintptr_t)w & 15)) return asb::fail("head_matmul_mma: K = %d must be a multiple of 8 and w 16-byte aligned", K);
  if (H > 65535 || (N + HB - 1) / HB > 65535) return asb::fail("head_matmul_mma: %d heads of %d columns exceed the grid", H, N);
  dim3 grid((T + HB - 1) / HB, H, (N + HB - 1) / HB);
  using B = __nv_bfloat16;
  if (x_f32 && out_f32)
    asb::launch(head_matmul_mma_kernel<float, float>, grid, 128, 0, stream, (float*)out, out_row, out_head, (const float*)x, x_row, x_head, (const B*)w, (const B*)gate, gate_row, T, K, N);
  else if (x_f32)
    asb::launch(head_matmul_mma_kernel<float, B>, grid, 128, 0, stream, (B*)out, out_row, out_head, (const float*)x, x_row, x_head, (const B*)w, (const B*)gate, gate_row, T, K, N);
  else if (out_f32)
    asb::launch(head_matmul_mma_kernel<B, float>, grid, 128, 0, stream, (float*)out, out_row, out_head, (const B*)x, x_row, x_head, (const B*)w, (const B*)gate, gate_row, T, K, N);
  else
    asb::launch(head_matmul_mma_kernel<B, B>, grid, 128, 0, stream, (B*)out, out_row, out_head, (const B*)x, x_row, x_head, (const B*)w, (const B*)gate, gate_row, T, K, N);
  return asb::check_launch("head_matmul_mma");
}

namespace {

template <int NT>
int launch_attention(const LatentParams& p, int num_tokens, size_t smem, cudaStream_t stream) {
  auto kern = latent_attention_mma_kernel<NT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return asb::fail("latent_attention_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
  dim3 grid((num_tokens + p.QT - 1) / p.QT + p.R, p.HC, p.NP);
  asb::launch(kern, grid, kWarps * 32, smem, stream, p);
  return asb::check_launch("latent_attention_mma");
}

size_t smem_bytes(int LDK) {
  return sizeof(__nv_bfloat16) * ((size_t)(MR + 2 * KT) * LDK + MR * LDP) + sizeof(float) * (MR * LDS + 3 * MR);
}

int padded_key_stride(int rank, int rot) {
  const int dkp = (rank + rot + 15) / 16 * 16;
  int nt = 1;
  while (64 * nt < rank) nt <<= 1;
  const int widest = dkp > 64 * nt ? dkp : 64 * nt;  // the value columns a warp reads may lie beyond Dk
  return widest + 8;
}

}  // namespace

extern "C" int asb_latent_attention_mma_supported(int rank, int rot) {
  return rank >= 1 && rank <= 512 && smem_bytes(padded_key_stride(rank, rot)) <= 220 * 1024;
}

extern "C" void asb_latent_attention_mma_tile_shape(int H, int* QT, int* GC) {
  *GC = H < MR ? H : MR;
  *QT = MR / *GC;
}

extern "C" int asb_latent_attention_mma(float* out, const float* q, const void* pages, const int* block_tables,
                                        const int* req_q_start, const int* req_pos_start, float* part_m, float* part_l,
                                        float* part_acc, int num_tokens, int R, int H, int rank, int rot, int bs,
                                        int table_width, int PS, int NP, float scale, int window, cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (!asb_latent_attention_mma_supported(rank, rot)) return asb::fail("latent_attention_mma: latent %d + %d is not taken", rank, rot);
  if (NP < 1 || PS < KT || PS % KT) return asb::fail("latent_attention_mma: partition size %d must be a positive multiple of %d", PS, KT);
  if (NP > 1 && (!part_m || !part_l || !part_acc)) return asb::fail("latent_attention_mma: %d partitions need scratch", NP);
  if (NP > 65535) return asb::fail("latent_attention_mma: %d partitions exceed the grid", NP);
  LatentParams p;
  p.q = q; p.out = out; p.pages = (const __nv_bfloat16*)pages; p.block_tables = block_tables;
  p.req_q_start = req_q_start; p.req_pos_start = req_pos_start; p.part_m = part_m; p.part_l = part_l; p.part_acc = part_acc;
  p.R = R; p.H = H; p.rank = rank; p.Dk = rank + rot; p.DKP = (p.Dk + 15) / 16 * 16; p.LDK = padded_key_stride(rank, rot);
  p.bs = bs; p.table_width = table_width;
  asb_latent_attention_mma_tile_shape(H, &p.QT, &p.GC);
  p.HC = (H + p.GC - 1) / p.GC;
  p.PS = PS; p.NP = NP; p.scale = scale; p.window = window;
  const size_t smem = smem_bytes(p.LDK);
  if (rank <= 64) return launch_attention<1>(p, num_tokens, smem, stream);
  if (rank <= 128) return launch_attention<2>(p, num_tokens, smem, stream);
  if (rank <= 256) return launch_attention<4>(p, num_tokens, smem, stream);
  return launch_attention<8>(p, num_tokens, smem, stream);
}
