// Kernels around a selective state-space recurrence with a scalar decay per head (the form
// S_t = exp(-exp(A_h) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D_h x_t). The recurrence
// itself runs asb_linear_recurrence_shared (k = B, q = C, v = x, a decay and an input weight per
// token, groups of heads sharing B and C); here is what comes before and after it:
//
//   asb_conv_steps         a causal convolution per channel over a request's tokens, with bias and
//                          SiLU: out[t, c] = silu(b_c + sum_j w[c, j] in[t - (K - 1) + j, c]), the
//                          inputs before a portion's first token read from the request's state
//                          (the last K - 1 inputs of what came before; zeros for a new request).
//                          In the same launch, per head: dt = softplus(z + dt_bias_h), the token's
//                          decay exp(-exp(A_h) dt) and input weight dt, all float32.
//   asb_conv_state_update  the state after the step: the last K - 1 inputs of each request
//                          (a portion shorter than that shifts what the state held).
//   asb_gate_group_norm    (y + D_h x) silu(z), RMS-normed in equal parts of the row (each part by
//                          its own root mean square), times a gain: the gate comes before the norm.
//
// Taps, biases, dt_bias, A and D are float32 arrays; inputs and outputs are in the compute dtype;
// everything between is float32 and each stored value is rounded once.
#include "common.cuh"

namespace {

constexpr int kConvThreads = 128;
constexpr int kConvTokens = 32;
constexpr int kConvWindow = 8;  // taps up to which a thread keeps the convolution's window in registers

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct ConvParams {
  void* out;               // [T, C]
  float* decay;            // [T, H]
  float* weight;           // [T, H]
  const void* proj;        // [T, stride]
  const float* taps;       // [C, K]
  const float* bias;       // [C]
  const float* conv_state; // [slots, K - 1, C]
  const float* dt_bias;    // [H]
  const float* a_log;      // [H]
  const int* state_slots;  // [R]
  const int* req_q_start;  // [R + 1]
  int stride, conv_off, dt_off, C, K, H, R;
};

// V neighbouring channels of one token in one load or store (V = 2 where every row's channels start at an
// even element: half as many memory instructions, each twice as wide).
template <typename T, int V> struct Lanes;
template <typename T> struct Lanes<T, 1> {
  static __device__ __forceinline__ void load(const T* at, float* v) { v[0] = asb::to_float(*at); }
  static __device__ __forceinline__ void store(T* at, const float* v) { *at = asb::from_float<T>(v[0]); }
};
template <> struct Lanes<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* at, float* v) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(at));
    v[0] = f.x; v[1] = f.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* at, const float* v) {
    *reinterpret_cast<__nv_bfloat162*>(at) = __floats2bfloat162_rn(v[0], v[1]);
  }
};
template <> struct Lanes<float, 2> {
  static __device__ __forceinline__ void load(const float* at, float* v) {
    const float2 f = *reinterpret_cast<const float2*>(at);
    v[0] = f.x; v[1] = f.y;
  }
  static __device__ __forceinline__ void store(float* at, const float* v) { *reinterpret_cast<float2*>(at) = make_float2(v[0], v[1]); }
};

// grid.x: token tiles of all requests (a block finds its request by bisection), grid.y: chunks of 128
// columns: the C / V groups of V neighbouring channels, then the H step columns.
template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads)
conv_steps_kernel(const ConvParams p) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  // request r's tiles are the blocks from first_r = req_q_start[r] / kConvTokens + r on: first_(r+1) - first_r
  // is at least the tiles r needs, so the ranges do not meet, and the last is below the grid's
  // tokens / kConvTokens + R. The block's request: the last r with first_r <= blockIdx.x, by bisection.
  int lo = 0, hi = p.R - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (p.req_q_start[mid] / kConvTokens + mid <= (int)blockIdx.x) lo = mid;
    else hi = mid - 1;
  }
  const int r = lo, row_lo = p.req_q_start[r], q_len = p.req_q_start[r + 1] - row_lo;
  const int tile = blockIdx.x - (row_lo / kConvTokens + r);
  if (tile < 0 || tile * kConvTokens >= q_len) return;
  const int column = blockIdx.y * kConvThreads + threadIdx.x;
  if (column >= p.C / V + p.H) return;
  const int q0 = tile * kConvTokens, nq = min(kConvTokens, q_len - q0);
  const T* proj = (const T*)p.proj;
  if (column >= p.C / V) {
    const int h = column - p.C / V;
    const float bias = p.dt_bias[h], rate = expf(p.a_log[h]);
    for (int q = q0; q < q0 + nq; ++q) {
      const size_t row = (size_t)(row_lo + q);
      const float dt = softplus_f(asb::to_float(proj[row * p.stride + p.dt_off + h]) + bias);
      p.decay[row * p.H + h] = expf(-rate * dt);
      p.weight[row * p.H + h] = dt;
    }
    return;
  }
  const int K = p.K, c = column * V;
  const float* w = p.taps + (size_t)c * K;  // channel c + v's taps: w[v * K ..]
  const float* held = p.conv_state + (size_t)p.state_slots[r] * (K - 1) * p.C + c;
  const T* in = proj + p.conv_off + c;
  T* out = (T*)p.out;
  float b[V];
#pragma unroll
  for (int v = 0; v < V; ++v) b[v] = p.bias[c + v];
  if (K <= kConvWindow) {
    // Up to kConvWindow taps: the taps padded in front with zeros to kConvWindow (a zero tap leaves the
    // sum as it is, so the sum runs in the same order as below), the last kConvWindow - 1 inputs kept in
    // registers, and kConvWindow tokens at a time: their loads are in flight together, and each input
    // is read once.
    float w8[kConvWindow][V], hist[kConvWindow - 1][V];
#pragma unroll
    for (int j = 0; j < kConvWindow; ++j)
#pragma unroll
      for (int v = 0; v < V; ++v) w8[j][v] = j >= kConvWindow - K ? w[v * K + j - (kConvWindow - K)] : 0.f;
#pragma unroll
    for (int i = 0; i < kConvWindow - 1; ++i) {
      const int at = q0 - (kConvWindow - 1) + i;  // negative: before the portion, K - 1 of them in the state
      if (at >= 0) {
        Lanes<T, V>::load(in + (size_t)(row_lo + at) * p.stride, hist[i]);
      } else if (K - 1 + at >= 0) {
        Lanes<float, V>::load(held + (size_t)(K - 1 + at) * p.C, hist[i]);
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) hist[i][v] = 0.f;
      }
    }
    for (int q = q0; q < q0 + nq; q += kConvWindow) {
      float x[2 * kConvWindow - 1][V];
#pragma unroll
      for (int i = 0; i < kConvWindow - 1; ++i)
#pragma unroll
        for (int v = 0; v < V; ++v) x[i][v] = hist[i][v];
#pragma unroll
      for (int i = 0; i < kConvWindow; ++i) {
        if (q + i < q0 + nq) {
          Lanes<T, V>::load(in + (size_t)(row_lo + q + i) * p.stride, x[kConvWindow - 1 + i]);
        } else {
#pragma unroll
          for (int v = 0; v < V; ++v) x[kConvWindow - 1 + i][v] = 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < kConvWindow; ++i) {
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          acc[v] = b[v];
#pragma unroll
          for (int j = 0; j < kConvWindow; ++j) acc[v] = fmaf(w8[j][v], x[i + j][v], acc[v]);
          acc[v] = silu_f(acc[v]);
        }
        if (q + i < q0 + nq) Lanes<T, V>::store(out + (size_t)(row_lo + q + i) * p.C + c, acc);
      }
#pragma unroll
      for (int i = 0; i < kConvWindow - 1; ++i)
#pragma unroll
        for (int v = 0; v < V; ++v) hist[i][v] = x[kConvWindow + i][v];
    }
    return;
  }
  for (int v = 0; v < V; ++v) {
    for (int q = q0; q < q0 + nq; ++q) {
      float acc = b[v];
      for (int j = 0; j < K; ++j) {
        const int at = q - (K - 1) + j;  // input index within the portion; negative: before it
        const float x = at >= 0 ? asb::to_float(in[(size_t)(row_lo + at) * p.stride + v]) : held[(size_t)(K - 1 + at) * p.C + v];
        acc = fmaf(w[v * K + j], x, acc);
      }
      out[(size_t)(row_lo + q) * p.C + c + v] = asb::from_float<T>(silu_f(acc));
    }
  }
}

template <typename T>
__global__ void conv_state_update_kernel(float* __restrict__ conv_state, const T* __restrict__ proj, int stride, int conv_off,
                                         const int* __restrict__ state_slots, const int* __restrict__ req_q_start, int C, int K) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row_lo = req_q_start[r], n = req_q_start[r + 1] - row_lo;
  float* held = conv_state + (size_t)state_slots[r] * (K - 1) * C + c;
  // entry s of the new state is input n - (K - 1) + s of the portion; a negative index is what the old
  // state held at s + n (read before any entry at or above it is written: s rises)
  for (int s = 0; s < K - 1; ++s) {
    const int at = n - (K - 1) + s;
    held[(size_t)s * C] = at >= 0 ? asb::to_float(proj[(size_t)(row_lo + at) * stride + conv_off + c]) : held[(size_t)(s + n) * C];
  }
}

// One block per (token, part of the row).
template <typename T>
__global__ void gate_group_norm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ x, int x_stride,
                                       const T* __restrict__ z, int z_stride, const float* __restrict__ skip,
                                       const float* __restrict__ gain, int width, int part_width, int head_width, float eps) {
  extern __shared__ float vals[];
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * part_width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part_width; i += blockDim.x) {
    const int c = c0 + i;
    float v = y[t * width + c];
    if (skip) v = fmaf(skip[c / head_width], asb::to_float(x[t * x_stride + c]), v);
    v *= silu_f(asb::to_float(z[t * z_stride + c]));
    vals[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) / (float)part_width + eps);
  for (int i = threadIdx.x; i < part_width; i += blockDim.x) {
    const int c = c0 + i;
    out[t * width + c] = asb::from_float<T>(vals[i] * inv * gain[c]);  // (each thread reads back what it wrote)
  }
}

}  // namespace

extern "C" int asb_conv_steps(void* out, float* decay, float* weight, const void* proj, int stride, int conv_off, int dt_off,
                              const float* taps, const float* bias, const float* conv_state, const float* dt_bias,
                              const float* a_log, const int* state_slots, const int* req_q_start, int num_tokens, int R,
                              int C, int K, int H, int dtype, cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (K < 1 || K > 64) return asb::fail("conv_steps: %d taps", K);
  ConvParams p;
  p.out = out; p.decay = decay; p.weight = weight; p.proj = proj; p.taps = taps; p.bias = bias; p.conv_state = conv_state;
  p.dt_bias = dt_bias; p.a_log = a_log; p.state_slots = state_slots; p.req_q_start = req_q_start;
  p.stride = stride; p.conv_off = conv_off; p.dt_off = dt_off; p.C = C; p.K = K; p.H = H; p.R = R;
  // two channels a thread where every row's channels start at an even element (and so at 4 or 8 bytes)
  const int esize = dtype == asb::kFloat32 ? 4 : 2;
  const bool two = C % 2 == 0 && conv_off % 2 == 0 && stride % 2 == 0 && K <= kConvWindow &&
                   ((uintptr_t)proj % (2 * esize)) == 0 && ((uintptr_t)out % (2 * esize)) == 0 && ((uintptr_t)conv_state % 8) == 0;
  const int V = two ? 2 : 1;
  dim3 grid((num_tokens + kConvTokens - 1) / kConvTokens + R, (C / V + H + kConvThreads - 1) / kConvThreads);
  if (two) {
    ASB_DISPATCH_DTYPE(dtype, T, asb::launch(conv_steps_kernel<T, 2>, grid, kConvThreads, 0, stream, p));
  } else {
    ASB_DISPATCH_DTYPE(dtype, T, asb::launch(conv_steps_kernel<T, 1>, grid, kConvThreads, 0, stream, p));
  }
  return asb::check_launch("conv_steps");
}

extern "C" int asb_conv_state_update(float* conv_state, const void* proj, int stride, int conv_off, const int* state_slots,
                                     const int* req_q_start, int R, int C, int K, int dtype, cudaStream_t stream) {
  if (R == 0 || K < 2) return 0;
  dim3 grid(R, (C + 127) / 128);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(conv_state_update_kernel<T>, grid, 128, 0, stream, conv_state, (const T*)proj,
                                           stride, conv_off, state_slots, req_q_start, C, K));
  return asb::check_launch("conv_state_update");
}

// y: float32 [T, width]; x (may be null with skip null) and z: the compute dtype with their row
// strides; skip [width / head_width]; gain [width]; `parts` equal parts of the row normed one by one.
extern "C" int asb_gate_group_norm(void* out, const float* y, const void* x, int x_stride, const void* z, int z_stride,
                                   const float* skip, const float* gain, int num_tokens, int width, int parts,
                                   int head_width, float eps, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (parts < 1 || width % parts || head_width < 1 || width % head_width) return asb::fail("gate_group_norm: %d columns in %d parts, heads of %d", width, parts, head_width);
  const int part_width = width / parts;
  const size_t smem = sizeof(float) * part_width;
  if (smem > 200 * 1024 || parts > 65535) return asb::fail("gate_group_norm: parts of %d columns", part_width);
  const int threads = part_width >= 1024 ? 256 : (part_width >= 256 ? 128 : 64);
  dim3 grid(num_tokens, parts);
#define ASB_GGN(T)                                                                                                       \
  {                                                                                                                      \
    auto kern = gate_group_norm_kernel<T>;                                                                               \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
    if (e != cudaSuccess) return asb::fail("gate_group_norm: shared memory %zu: %s", smem, cudaGetErrorString(e));       \
    asb::launch(kern, grid, threads, smem, stream, (T*)out, y, (const T*)x, x_stride, (const T*)z, z_stride, skip, gain, \
                width, part_width, head_width, eps);                                                                     \
  }
  ASB_DISPATCH_DTYPE(dtype, T, ASB_GGN(T));
#undef ASB_GGN
  return asb::check_launch("gate_group_norm");
}
