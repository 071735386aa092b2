// Routed experts: selection, grouping of the step's (token, expert) pairs by expert, the
// experts' products over the grouped rows, and the weighted sum back per token.
//
//   asb_moe_route     z [T, stride] float32 router logits -> the chosen experts and their weights.
//                     Scores s = sigmoid(z) (or softmax over the experts, `softmax` 1). With G > 1
//                     groups of neighbouring experts, a group's score is the sum of its `group_top`
//                     largest scores and only experts of the `keep` best groups can be chosen. The
//                     `top` largest allowed scores win (ties: the lower index); their weights are
//                     s / (sum s + 1e-20) * scale (`renorm` 0: s * scale). Column `gate_col` of z,
//                     if not negative, gives sigmoid(z) per token: the gate of a shared expert.
//   asb_moe_group     pairs sorted by expert: offsets [E + 1], the token of each sorted row, and
//                     for each (token, choice) its sorted row
//   asb_moe_glu       hidden[row] = act(x[token] . gate_e^T, x[token] . up_e^T) for the rows of
//                     each expert e: g = min(., limit), u = clamp(., -limit, limit),
//                     g sigmoid(slope g) (u + shift); limit <= 0: no clamping
//   asb_moe_down      y[row] = hidden[row] . down_e^T, float32
//   asb_moe_combine   out[t] = sum_k weight[t, k] y[row(t, k)] (+ shared_gate[t] * shared[t]), float32,
//                     the choices added in their order of selection
//
// The products run on CUDA cores with float32 multiply-adds for both element types, every
// output element summed in an order that depends on k alone (chains of fused multiply-adds over
// runs of 256 consecutive k, the runs added in order), so a row's result does not depend on
// which rows share its tile. Router arithmetic is float32.
#include "common.cuh"

namespace {

// ---- selection ----------------------------------------------------------------------------

struct RouteParams {
  const float* z;
  int stride, E, G, group_top, keep, top, gate_col, softmax, renorm;
  float scale;
  int* ids;        // [T, top]
  float* weights;  // [T, top]
  float* shared_gate;  // [T] or null
  const float* bias;   // [E] or null: added to the scores for the final choice only, not to the weights
};

// one warp per token; scores and masks in shared memory
__global__ void moe_route_kernel(const RouteParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ float sm[];
  float* s = sm;                 // [E] scores
  float* allowed = s + p.E;      // [E] 1 / 0
  float* gs = allowed + p.E;     // [G] group scores
  const int t = blockIdx.x, lane = threadIdx.x;
  const float* z = p.z + (size_t)t * p.stride;
  if (p.softmax) {
    float mx = -INFINITY;
    for (int e = lane; e < p.E; e += 32) mx = fmaxf(mx, z[e]);
    mx = asb::warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < p.E; e += 32) sum += expf(z[e] - mx);
    sum = asb::warp_sum(sum);
    for (int e = lane; e < p.E; e += 32) s[e] = expf(z[e] - mx) / sum;
  } else {
    for (int e = lane; e < p.E; e += 32) s[e] = 1.f / (1.f + expf(-z[e]));
  }
  for (int e = lane; e < p.E; e += 32) allowed[e] = 1.f;
  __syncwarp();
  if (p.G > 1) {
    const int per = p.E / p.G;
    for (int g = lane; g < p.G; g += 32) {
      // sum of the group's `group_top` largest scores, by repeated selection
      float total = 0.f, last = INFINITY;
      int last_at = -1;
      for (int n = 0; n < p.group_top && n < per; ++n) {
        float best = -INFINITY;
        int at = -1;
        for (int e = 0; e < per; ++e) {
          const float v = s[g * per + e];
          const bool after = v < last || (v == last && e > last_at);  // strictly behind the one taken before
          if (after && v > best) { best = v; at = e; }
        }
        total += best;
        last = best;
        last_at = at;
      }
      gs[g] = total;
    }
    __syncwarp();
    for (int e = lane; e < p.E; e += 32) allowed[e] = 0.f;
    __syncwarp();
    for (int n = 0; n < p.keep; ++n) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < p.G; g += 32)
        if (gs[g] > best) { best = gs[g]; at = g; }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at == 0x7fffffff) break;
      for (int e = lane; e < per; e += 32) allowed[at * per + e] = 1.f;
      if (lane == 0) gs[at] = -INFINITY;
      __syncwarp();
    }
  }
  float sum = 0.f;
  float mine = 0.f;  // lane k keeps the k-th chosen score
  int mine_at = 0;
  for (int n = 0; n < p.top; ++n) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < p.E; e += 32) {
      const float c = p.bias ? s[e] + p.bias[e] : s[e];
      if (allowed[e] > 0.f && c > best) { best = c; at = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) { at = 0; best = 0.f; }  // fewer allowed experts than `top`: weight 0
    else {
      best = s[at];  // the weight is the score itself
      if (lane == 0) allowed[at] = 0.f;
    }
    __syncwarp();
    sum += best;
    if ((n & 31) == lane) {
      // (top <= 32 is checked on the host)
      mine = best;
      mine_at = at;
    }
  }
  if (lane < p.top) {
    p.ids[(size_t)t * p.top + lane] = mine_at;
    p.weights[(size_t)t * p.top + lane] = (p.renorm ? mine / (sum + 1e-20f) : mine) * p.scale;
  }
  if (p.shared_gate && p.gate_col >= 0 && lane == 0) p.shared_gate[t] = 1.f / (1.f + expf(-z[p.gate_col]));
}

// ---- grouping -----------------------------------------------------------------------------

// One block. counts and cursors in shared memory (E <= 4096).
__global__ void moe_group_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ offsets,
                                 int* __restrict__ row_token, int* __restrict__ pair_row, int top) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ int cnt[];  // [E] counts, then [E] cursors
  int* cursor = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += cnt[e];
    }
    offsets[E] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int at = atomicAdd(&cursor[ids[i]], 1);
    row_token[at] = i / top;
    pair_row[i] = at;
  }
}

// ---- products over grouped rows -----------------------------------------------------------

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kChunk = 256;

struct GroupedParams {
  void* out;             // [rows, N]
  const void* x;         // GLU: [T, K] by token; else [rows, K]
  const int* row_token;  // GLU only
  const int* offsets;    // [E + 1]
  const void* w;         // [E, N, K]
  const void* w2;        // GLU: the up matrices
  int E, N, K;
  float limit, slope, shift;
};

template <typename TIn, typename TOut, bool GLU>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const GroupedParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ float us[GLU ? BK : 1][BN + 4];
  __shared__ int src_row[BM];
  // which expert and which tile of its rows?
  int tile = blockIdx.y, e = 0, begin = 0, count = 0;
  for (; e < p.E; ++e) {
    begin = p.offsets[e];
    count = p.offsets[e + 1] - begin;
    const int tiles = (count + BM - 1) / BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e == p.E) return;
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  const int rows = min(BM, count - m0);
  const int tid = threadIdx.x;
  if (tid < BM) src_row[tid] = tid < rows ? (GLU ? p.row_token[begin + m0 + tid] : begin + m0 + tid) : -1;
  __syncthreads();
  const int tx = tid % 16, ty = tid / 16;
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  const int K = p.K, N = p.N;
  const TIn* x = (const TIn*)p.x;
  const TIn* w = (const TIn*)p.w + (size_t)e * N * K;
  const TIn* w2 = GLU ? (const TIn*)p.w2 + (size_t)e * N * K : nullptr;
  const int xrow = src_row[lrow];

  float acc[TM][TN], total[TM][TN], acc2[GLU ? TM : 1][TN], total2[GLU ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = total[i][j] = 0.f;
      if constexpr (GLU) acc2[i][j] = total2[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int wn = n0 + lrow;
      xs[lk + u][lrow] = (xrow >= 0 && k < K) ? asb::to_float(x[(size_t)xrow * K + k]) : 0.f;
      ws[lk + u][lrow] = (wn < N && k < K) ? asb::to_float(w[(size_t)wn * K + k]) : 0.f;
      if constexpr (GLU) us[lk + u][lrow] = (wn < N && k < K) ? asb::to_float(w2[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN], c[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b[j] = ws[kk][tx * TN + j];
        if constexpr (GLU) c[j] = us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if constexpr (GLU) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
        }
    }
    __syncthreads();
    if ((k0 + BK) % kChunk == 0 || k0 + BK >= K) {
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          total[i][j] += acc[i][j];
          acc[i][j] = 0.f;
          if constexpr (GLU) {
            total2[i][j] += acc2[i][j];
            acc2[i][j] = 0.f;
          }
        }
    }
  }
  TOut* out = (TOut*)p.out;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= rows) continue;
    const size_t orow = (size_t)(begin + m0 + m) * N;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = total[i][j];
      if constexpr (GLU) {
        float g = v, u = total2[i][j];
        if (p.limit > 0.f) {
          g = fminf(g, p.limit);
          u = fminf(fmaxf(u, -p.limit), p.limit);
        }
        v = g / (1.f + expf(-p.slope * g)) * (u + p.shift);
      }
      out[orow + n] = asb::from_float<TOut>(v);
    }
  }
}

// ---- weighted sum back per token ----------------------------------------------------------

// ids, x, experts: where ids is given, a choice of index >= experts is an identity expert, whose
// output is the token's own input row x[t] (no row of y belongs to it).
template <typename T, typename TX>
__global__ void moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const int* __restrict__ pair_row,
                                   const float* __restrict__ weights, const T* __restrict__ shared,
                                   const float* __restrict__ shared_gate, int top, int N,
                                   const int* __restrict__ ids, const TX* __restrict__ x, int experts) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t pair = (size_t)t * top + k;
      const float v = ids && ids[pair] >= experts ? asb::to_float(x[(size_t)t * N + n]) : y[(size_t)pair_row[pair] * N + n];
      sum = fmaf(weights[pair], v, sum);
    }
    if (shared) {
      const float sv = asb::to_float(shared[(size_t)t * N + n]);
      sum = shared_gate ? fmaf(shared_gate[t], sv, sum) : sum + sv;
    }
    out[(size_t)t * N + n] = sum;
  }
}

int row_tiles(int pairs, int E) { return pairs / BM + (pairs < E ? pairs : E); }

}  // namespace

extern "C" int asb_moe_route_biased(const float* z, int stride, int T, int E, int G, int group_top, int keep, int top,
                                    int gate_col, int softmax, int renorm, float scale, const float* bias, int* ids,
                                    float* weights, float* shared_gate, cudaStream_t stream) {
  if (T == 0) return 0;
  if (E < 1 || top < 1 || top > 32 || top > E) return asb::fail("moe_route: top %d of %d experts (at most 32)", top, E);
  if (G < 1 || E % G || keep < 1 || keep > G) return asb::fail("moe_route: %d experts in %d groups, %d kept", E, G, keep);
  if ((size_t)(2 * E + G) * 4 > 48 * 1024) return asb::fail("moe_route: %d experts are too many", E);
  RouteParams p;
  p.z = z; p.stride = stride; p.E = E; p.G = G; p.group_top = group_top; p.keep = keep; p.top = top;
  p.gate_col = gate_col; p.softmax = softmax; p.renorm = renorm; p.scale = scale;
  p.ids = ids; p.weights = weights; p.shared_gate = shared_gate; p.bias = bias;
  asb::launch(moe_route_kernel, T, 32, sizeof(float) * (2 * E + G), stream, p);
  return asb::check_launch("moe_route");
}

extern "C" int asb_moe_route(const float* z, int stride, int T, int E, int G, int group_top, int keep, int top,
                             int gate_col, int softmax, int renorm, float scale, int* ids, float* weights,
                             float* shared_gate, cudaStream_t stream) {
  return asb_moe_route_biased(z, stride, T, E, G, group_top, keep, top, gate_col, softmax, renorm, scale, nullptr, ids,
                              weights, shared_gate, stream);
}

extern "C" int asb_moe_group(const int* ids, int T, int top, int E, int* offsets, int* row_token, int* pair_row,
                             cudaStream_t stream) {
  if (T == 0) return 0;
  if (E > 4096) return asb::fail("moe_group: %d experts exceed 4096", E);
  asb::launch(moe_group_kernel, 1, 1024, sizeof(int) * 2 * E, stream, ids, T * top, E, offsets, row_token, pair_row, top);
  return asb::check_launch("moe_group");
}

extern "C" int asb_moe_glu(void* hidden, const void* x, const int* row_token, const int* offsets, const void* gate,
                           const void* up, int pairs, int E, int F, int K, float limit, float slope, float shift,
                           int dtype, cudaStream_t stream) {
  if (pairs == 0) return 0;
  GroupedParams p;
  p.out = hidden; p.x = x; p.row_token = row_token; p.offsets = offsets; p.w = gate; p.w2 = up;
  p.E = E; p.N = F; p.K = K; p.limit = limit; p.slope = slope; p.shift = shift;
  dim3 grid((F + BN - 1) / BN, row_tiles(pairs, E));
  if (grid.y > 65535) return asb::fail("moe_glu: %d rows exceed the grid", pairs);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(grouped_gemm_kernel<T, T, true>, grid, 256, 0, stream, p));
  return asb::check_launch("moe_glu");
}

extern "C" int asb_moe_down(float* y, const void* hidden, const int* offsets, const void* down, int pairs, int E,
                            int N, int F, int dtype, cudaStream_t stream) {
  if (pairs == 0) return 0;
  GroupedParams p;
  p.out = y; p.x = hidden; p.row_token = nullptr; p.offsets = offsets; p.w = down; p.w2 = nullptr;
  p.E = E; p.N = N; p.K = F; p.limit = 0.f; p.slope = 1.f; p.shift = 0.f;
  dim3 grid((N + BN - 1) / BN, row_tiles(pairs, E));
  if (grid.y > 65535) return asb::fail("moe_down: %d rows exceed the grid", pairs);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(grouped_gemm_kernel<T, float, false>, grid, 256, 0, stream, p));
  return asb::check_launch("moe_down");
}

// ids [T, top], x [T, N] in x_dtype, experts: null / 0 for a layer without identity experts.
extern "C" int asb_moe_combine_identity(float* out, const float* y, const int* pair_row, const float* weights,
                                        const void* shared, const float* shared_gate, int T, int top, int N, int dtype,
                                        const int* ids, const void* x, int x_dtype, int experts, cudaStream_t stream) {
  if (T == 0) return 0;
  if (ids && !x) return asb::fail("moe_combine: identity experts need the tokens' input rows");
  const int threads = N >= 1024 ? 256 : 128;
  ASB_DISPATCH_DTYPE(dtype, T_, {
    if (x_dtype == asb::kFloat32)
      asb::launch(moe_combine_kernel<T_, float>, T, threads, 0, stream, out, y, pair_row, weights, (const T_*)shared,
                  shared_gate, top, N, ids, (const float*)x, experts);
    else
      asb::launch(moe_combine_kernel<T_, __nv_bfloat16>, T, threads, 0, stream, out, y, pair_row, weights,
                  (const T_*)shared, shared_gate, top, N, ids, (const __nv_bfloat16*)x, experts);
  });
  return asb::check_launch("moe_combine");
}

extern "C" int asb_moe_combine(float* out, const float* y, const int* pair_row, const float* weights,
                               const void* shared, const float* shared_gate, int T, int top, int N, int dtype,
                               cudaStream_t stream) {
  return asb_moe_combine_identity(out, y, pair_row, weights, shared, shared_gate, T, top, N, dtype, nullptr, nullptr, 0, 0,
                                  stream);
}
