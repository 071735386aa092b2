// Softmax attention over a cached low-rank latent. Per token the cache holds one vector
// [c | kr]: c, the RMS-normed latent of `rank` values from which every head's keys and values
// are up-projections (k_h = Wuk_h c, v_h = Wuv_h c), and kr, `rot` values of a position-encoded
// key part that all heads share. The up-projections are moved to the query side, so that the
// cache is read as it is:
//
//   score_h(t, j) = (Wuk_h^T q_h(t)) . c_j + qr_h(t) . kr_j         (times scale)
//   out_h(t)      = Wuv_h (sum_j p_h(t, j) c_j)
//
// i.e. attention with one shared key head of width rank + rot whose values are the first `rank`
// entries of the keys. Three kernels:
//
//   asb_latent_prepare    per token: norm the latent, turn kr by the token's position, write
//                         [c | kr] to the token's cache slot; turn each head's qr and put it
//                         behind that head's absorbed query in q_lat (float32)
//   asb_head_matmul       out[t, h, :] = x[t, h, :] . w[h] per head (w[h]: [K, N]), optionally
//                         times sigmoid(gate[t, h]): the query absorption and the value
//                         up-projection with the output gate
//   asb_latent_attention  the attention itself, for any mix of prompt portions and single
//                         tokens; float32 scores, weights and sums; key partitions aligned to
//                         absolute positions, merged by asb_attention_reduce
//
// The rotation pairs neighbours: of the first `rot_dims` entries, (2i, 2i + 1) turns by
// position * inv_freq[i]; angles are float32.
#include "common.cuh"

namespace {

// ---- prepare ------------------------------------------------------------------------------

struct PrepareParams {
  const void* proj;        // [T, stride]
  float* q_lat;            // [T, H, rank + rot]
  void* pages;             // [num_blocks, 1, bs, rank + rot]; null: nothing is stored
  const float* gain;       // [rank]
  const float* inv_freq;   // [rot_dims / 2]
  const int* positions;    // [T]
  const int* slots;        // [T]; negative: not stored
  int stride, q_off, kv_off;
  int H, D, rank, rot, rot_dims;
  float eps;
};

template <typename T>
__global__ void latent_prepare_kernel(const PrepareParams p) {
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = (const T*)p.proj + (size_t)t * p.stride;
  const float pos = (float)p.positions[t];
  const int Dk = p.rank + p.rot;
  // queries: each head's turned part, behind its absorbed part
  for (int i = threadIdx.x; i < p.H * p.rot; i += blockDim.x) {
    const int h = i / p.rot, e = i - h * p.rot;
    const T* qr = row + p.q_off + h * (p.D + p.rot) + p.D;
    float v = asb::to_float(qr[e]);
    if (e < p.rot_dims) {
      float s, c;
      sincosf(pos * p.inv_freq[e >> 1], &s, &c);
      const float other = asb::to_float(qr[e ^ 1]);
      v = (e & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
    }
    p.q_lat[((size_t)t * p.H + h) * Dk + p.rank + e] = v;
  }
  if (!p.pages) return;
  const int slot = p.slots[t];
  const T* kv = row + p.kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
    const float v = asb::to_float(kv[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) / (float)p.rank + p.eps);
  if (slot < 0) return;
  T* dst = (T*)p.pages + (size_t)slot * Dk;
  for (int i = threadIdx.x; i < p.rank; i += blockDim.x) dst[i] = asb::from_float<T>(asb::to_float(kv[i]) * inv * p.gain[i]);
  for (int e = threadIdx.x; e < p.rot; e += blockDim.x) {
    float v = asb::to_float(kv[p.rank + e]);
    if (e < p.rot_dims) {
      float s, c;
      sincosf(pos * p.inv_freq[e >> 1], &s, &c);
      const float other = asb::to_float(kv[p.rank + (e ^ 1)]);
      v = (e & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
    }
    dst[p.rank + e] = asb::from_float<T>(v);
  }
}

// ---- per-head products --------------------------------------------------------------------

constexpr int kHmTokens = 8;
constexpr int kHmThreads = 128;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(kHmThreads)
head_matmul_kernel(TO* __restrict__ out, int out_row, int out_head, const TX* __restrict__ x, int x_row, int x_head,
                   const TW* __restrict__ w, const TW* __restrict__ gate, int gate_row, int T, int K, int N) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ float xs[];  // [kHmTokens][K]
  const int t0 = blockIdx.x * kHmTokens, h = blockIdx.y;
  const int nt = min(kHmTokens, T - t0);
  for (int i = threadIdx.x; i < kHmTokens * K; i += kHmThreads) {
    const int t = i / K, k = i - t * K;
    xs[i] = t < nt ? asb::to_float(x[(size_t)(t0 + t) * x_row + (size_t)h * x_head + k]) : 0.f;
  }
  __syncthreads();
  const TW* wh = w + (size_t)h * K * N;
  for (int n = blockIdx.z * kHmThreads + threadIdx.x; n < N; n += gridDim.z * kHmThreads) {
    float acc[kHmTokens];
#pragma unroll
    for (int t = 0; t < kHmTokens; ++t) acc[t] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float wv = asb::to_float(wh[(size_t)k * N + n]);
#pragma unroll
      for (int t = 0; t < kHmTokens; ++t) acc[t] = fmaf(xs[t * K + k], wv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < kHmTokens; ++t) {
      if (t >= nt) break;
      float v = acc[t];
      if (gate) v /= 1.f + expf(-asb::to_float(gate[(size_t)(t0 + t) * gate_row + h]));
      out[(size_t)(t0 + t) * out_row + (size_t)h * out_head + n] = asb::from_float<TO>(v);
    }
  }
}

// ---- attention ----------------------------------------------------------------------------

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;
constexpr int kMaxRows = kWarps * kRowsPerWarp;  // 32 (token, head) rows a block
constexpr int kKeyTile = 32;

struct LatentParams {
  const float* q;            // [T, H, Dk], Dk = rank + rot
  float* out;                // [T, H, rank]
  const void* pages;         // [num_blocks, 1, bs, Dk]
  const int* block_tables;   // [R, table_width]
  const int* req_q_start;    // [R + 1]
  const int* req_pos_start;  // [R]
  float* part_m;             // [T, H, NP]        (NP > 1 only)
  float* part_l;
  float* part_acc;           // [T, H, NP, rank]
  int R, H, rank, Dk, bs, table_width;
  int QT, GC, HC;            // tokens per tile, heads per block, head chunks
  int PS, NP;
  float scale;
  int window;                // > 0: a query at p sees keys j with p - j < window only
};

template <typename T, int EPL>
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_kernel(const LatentParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ float smem[];
  const int Dk = p.Dk, Dv = p.rank;
  const int kstride = Dk | 1;  // odd stride: lanes reading one column of 32 keys hit 32 banks
  float* q_s = smem;                   // [32][Dk]
  float* k_s = q_s + kMaxRows * Dk;    // [32][kstride]; the values are its first Dv columns
  __shared__ int block_of_key[kKeyTile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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

  const int hi = pos0 + nq;  // exclusive
  const int part = blockIdx.z;
  // with a window no row of the tile sees a key before pos0 - window + 1 (pages before it may be gone)
  const int key_lo = max(part * p.PS, p.window > 0 ? pos0 - p.window + 1 : 0);
  const int key_hi = (int)min((long long)hi, (long long)(part + 1) * p.PS);

  for (int i = threadIdx.x; i < num_rows * Dk; i += blockDim.x) {
    const int rr = i / Dk, e = i - rr * Dk;
    const int qi = rr / gc, g = rr - qi * gc;
    q_s[rr * Dk + e] = p.q[((size_t)(row0 + qi) * p.H + head0 + g) * Dk + e] * p.scale;
  }

  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][EPL];
#pragma unroll
  for (int s = 0; s < kRowsPerWarp; ++s) {
    m[s] = -INFINITY;
    l[s] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[s][e] = 0.f;
  }
  const T* pages = (const T*)p.pages;
  const int* table = p.block_tables + (size_t)r * p.table_width;

  for (int kt0 = (key_lo / kKeyTile) * kKeyTile; kt0 < key_hi; kt0 += kKeyTile) {
    __syncthreads();
    if (threadIdx.x < kKeyTile) {
      const int j = kt0 + threadIdx.x;
      block_of_key[threadIdx.x] = (j >= key_lo && j < key_hi) ? table[j / p.bs] : -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kKeyTile * Dk; i += blockDim.x) {
      const int jj = i / Dk, e = i - jj * Dk;
      const int blk = block_of_key[jj];
      k_s[jj * kstride + e] = blk >= 0 ? asb::to_float(pages[((size_t)blk * p.bs + (kt0 + jj) % p.bs) * Dk + e]) : 0.f;
    }
    __syncthreads();
    const int j = kt0 + lane;
    const bool in_range = block_of_key[lane] >= 0;
#pragma unroll
    for (int s = 0; s < kRowsPerWarp; ++s) {
      const int rr = warp + s * kWarps;
      if (rr >= num_rows) break;
      const int pq = pos0 + rr / gc;
      const bool visible = in_range && j <= pq && (p.window <= 0 || pq - j < p.window);
      float score = -INFINITY;
      if (visible) {
        const float* qrow = q_s + rr * Dk;
        const float* krow = k_s + lane * kstride;
        float d = 0.f;
        for (int e = 0; e < Dk; ++e) d = fmaf(qrow[e], krow[e], d);
        score = d;
      }
      const float m_new = fmaxf(m[s], asb::warp_max(score));
      if (m_new == -INFINITY) continue;
      const float corr = expf(m[s] - m_new);
      const float pj = visible ? expf(score - m_new) : 0.f;
      l[s] = l[s] * corr + asb::warp_sum(pj);
      m[s] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[s][e] *= corr;
      for (int jj = 0; jj < kKeyTile; ++jj) {
        const float w = __shfl_sync(0xffffffffu, pj, jj);
        if (w == 0.f) continue;  // uniform across the warp
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          const int col = e * 32 + lane;
          if (col < Dv) acc[s][e] = fmaf(w, k_s[jj * kstride + col], acc[s][e]);
        }
      }
    }
  }

#pragma unroll
  for (int s = 0; s < kRowsPerWarp; ++s) {
    const int rr = warp + s * kWarps;
    if (rr >= num_rows) break;
    const int qi = rr / gc, g = rr - qi * gc;
    const size_t row = (size_t)(row0 + qi) * p.H + head0 + g;
    if (p.NP == 1) {
      const float inv = 1.f / l[s];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int col = e * 32 + lane;
        if (col < Dv) p.out[row * Dv + col] = acc[s][e] * inv;
      }
    } else {
      const size_t at = row * p.NP + blockIdx.z;
      if (lane == 0) {
        p.part_m[at] = m[s];
        p.part_l[at] = l[s];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int col = e * 32 + lane;
        if (col < Dv) p.part_acc[at * Dv + col] = acc[s][e];
      }
    }
  }
}

template <typename T, int EPL>
int launch_attention(const LatentParams& p, int num_tokens, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)kMaxRows * p.Dk + kKeyTile * (p.Dk | 1));
  auto kern = latent_attention_kernel<T, EPL>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return asb::fail("latent_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
  dim3 grid((num_tokens + p.QT - 1) / p.QT + p.R, p.HC, p.NP);
  asb::launch(kern, grid, kWarps * 32, smem, stream, p);
  return asb::check_launch("latent_attention");
}

}  // namespace

extern "C" int asb_latent_prepare(const void* proj, int stride, int q_off, int kv_off, float* q_lat, void* pages,
                                  const float* gain, const float* inv_freq, const int* positions, const int* slots,
                                  int T, int H, int D, int rank, int rot, int rot_dims, float eps, int dtype,
                                  cudaStream_t stream) {
  if (T == 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims < 0) return asb::fail("latent_prepare: %d turned entries of %d", rot_dims, rot);
  PrepareParams p;
  p.proj = proj; p.q_lat = q_lat; p.pages = pages; p.gain = gain; p.inv_freq = inv_freq;
  p.positions = positions; p.slots = slots; p.stride = stride; p.q_off = q_off; p.kv_off = kv_off;
  p.H = H; p.D = D; p.rank = rank; p.rot = rot; p.rot_dims = rot_dims; p.eps = eps;
  ASB_DISPATCH_DTYPE(dtype, T_, asb::launch(latent_prepare_kernel<T_>, T, 128, 0, stream, p));
  return asb::check_launch("latent_prepare");
}

// x: float32 (x_f32 1) or the compute dtype; out: float32 (out_f32 1) or the compute dtype; w and
// gate in the compute dtype.
extern "C" int asb_head_matmul(void* out, int out_f32, int out_row, int out_head, const void* x, int x_f32, int x_row,
                               int x_head, const void* w, const void* gate, int gate_row, int T, int H, int K, int N,
                               int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  if (H > 65535) return asb::fail("head_matmul: %d heads", H);
  const size_t smem = sizeof(float) * kHmTokens * K;
  if (smem > 200 * 1024) return asb::fail("head_matmul: K = %d is too long", K);
  dim3 grid((T + kHmTokens - 1) / kHmTokens, H, (N + kHmThreads - 1) / kHmThreads);
#define ASB_HM(TX, TO)                                                                                         \
  {                                                                                                            \
    auto kern = head_matmul_kernel<TX, TW, TO>;                                                                \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    if (e != cudaSuccess) return asb::fail("head_matmul: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    asb::launch(kern, grid, kHmThreads, smem, stream, (TO*)out, out_row, out_head, (const TX*)x, x_row, x_head, \
                (const TW*)w, (const TW*)gate, gate_row, T, K, N);                                             \
  }
  ASB_DISPATCH_DTYPE(dtype, TW, {
    if (x_f32 && out_f32) ASB_HM(float, float)
    else if (x_f32) ASB_HM(float, TW)
    else if (out_f32) ASB_HM(TW, float)
    else ASB_HM(TW, TW)
  });
#undef ASB_HM
  return asb::check_launch("head_matmul");
}

extern "C" int asb_latent_attention(float* out, const float* q, const void* pages, const int* block_tables,
                                    const int* req_q_start, const int* req_pos_start, float* part_m, float* part_l,
                                    float* part_acc, int num_tokens, int R, int H, int rank, int rot, int bs,
                                    int table_width, int PS, int NP, float scale, int window, int dtype,
                                    cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (rank < 1 || rank > 512) return asb::fail("latent_attention: latent size %d not in 1..512", rank);
  if (NP < 1 || PS < kKeyTile || PS % kKeyTile) return asb::fail("latent_attention: partition size %d must be a positive multiple of %d", PS, kKeyTile);
  if (NP > 1 && (!part_m || !part_l || !part_acc)) return asb::fail("latent_attention: %d partitions need scratch", NP);
  if (NP > 65535) return asb::fail("latent_attention: %d partitions exceed the grid", NP);
  LatentParams p;
  p.q = q; p.out = out; p.pages = pages; p.block_tables = block_tables; p.req_q_start = req_q_start;
  p.req_pos_start = req_pos_start; p.part_m = part_m; p.part_l = part_l; p.part_acc = part_acc;
  p.R = R; p.H = H; p.rank = rank; p.Dk = rank + rot; p.bs = bs; p.table_width = table_width;
  p.GC = H < kMaxRows ? H : kMaxRows;
  p.QT = kMaxRows / p.GC;
  p.HC = (H + p.GC - 1) / p.GC;
  p.PS = PS; p.NP = NP; p.scale = scale; p.window = window;
  if ((size_t)(kMaxRows * p.Dk + kKeyTile * (p.Dk | 1)) * 4 > 220 * 1024) return asb::fail("latent_attention: key width %d is too large", p.Dk);
  const int epl = (rank + 31) / 32;
#define ASB_LAT_CASE(E) case E: ASB_DISPATCH_DTYPE(dtype, T, return launch_attention<T, E>(p, num_tokens, stream)); break;
  switch (epl) {
    ASB_LAT_CASE(1) ASB_LAT_CASE(2) ASB_LAT_CASE(3) ASB_LAT_CASE(4) ASB_LAT_CASE(5) ASB_LAT_CASE(6) ASB_LAT_CASE(7) ASB_LAT_CASE(8)
    ASB_LAT_CASE(9) ASB_LAT_CASE(10) ASB_LAT_CASE(11) ASB_LAT_CASE(12) ASB_LAT_CASE(13) ASB_LAT_CASE(14) ASB_LAT_CASE(15) ASB_LAT_CASE(16)
  }
#undef ASB_LAT_CASE
  return 0;
}

// Query tile geometry for H heads: (tokens per tile, heads per block); the planner of the key
// partitions counts blocks with it.
extern "C" void asb_latent_attention_tile_shape(int H, int* QT, int* GC) {
  *GC = H < kMaxRows ? H : kMaxRows;
  *QT = kMaxRows / *GC;
}
