// Kernels for models whose layers add two sublayers that read the same stream,
// x <- x + mult (mixer(N1 x) + ff(N2 x)), over a float32 residual stream, and for what such a
// model does around its layers:
//
//   asb_residual_dual_norm   s = x + mult (y1 + y2) + bias (every term optional), written as the
//                            float32 stream, and N(s) gain1, N(s) gain2 in the compute dtype,
//                            N(s) = s / sqrt(mean(s^2) + eps): the sum of a layer and both norms of
//                            the next one in one pass over the row
//   asb_pair_embedding       x[t] = table[id[t]] + pairs[row(previous id, id[t])], float32: a
//                            hashed table of token pairs beside the token table. The id before a
//                            request's first token of the step is per-request state (0: none yet)
//   asb_concat_cast          [a ; b] per row in the compute dtype (the input of a product over
//                            two streams)
//
// Sums and norms are float32; each stored value is rounded once.
#include "common.cuh"

namespace {

int threads_for(int width) {
  int threads = 64;
  while (threads < width && threads < 1024) threads <<= 1;
  return threads;
}

// One block per row; the row's sum stays in shared memory between the two passes.
template <typename T>
__global__ void residual_dual_norm_kernel(float* __restrict__ out32, T* __restrict__ out1, T* __restrict__ out2,
                                          const float* __restrict__ x, const float* __restrict__ y1,
                                          const float* __restrict__ y2, const float* __restrict__ bias,
                                          const float* __restrict__ gain1, const float* __restrict__ gain2,
                                          int width, float mult, float eps) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const size_t at = (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = y1 ? y1[at + i] : 0.f;
    if (y2) y += y2[at + i];
    float s = x ? fmaf(mult, y, x[at + i]) : mult * y;
    if (bias) s += bias[i];
    row[i] = s;
    ss = fmaf(s, s, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float s = row[i];
    if (out32) out32[at + i] = s;
    const float n = s * inv;
    if (out1) out1[at + i] = asb::from_float<T>(n * gain1[i]);
    if (out2) out2[at + i] = asb::from_float<T>(n * gain2[i]);
  }
}

// One block per token. The block of a request's first token of the step reads the request's
// state (the id before it, plus one) and is the only one to write it (the request's last id of
// the step, plus one); every other token's predecessor is its neighbour in the flat batch.
template <typename T>
__global__ void pair_embedding_kernel(float* __restrict__ out, const T* __restrict__ table, const T* __restrict__ pairs,
                                      const int* __restrict__ ids, const int* __restrict__ positions,
                                      const int* __restrict__ req_q_start, const int* __restrict__ state_slots,
                                      int* __restrict__ last_id, int R, int width, int vocab, int buckets,
                                      int mul_prev, int mul_cur, int* __restrict__ status) {
  __shared__ int prev_s;
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = R;  // the request r with req_q_start[r] <= t < req_q_start[r + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (req_q_start[mid] <= t) lo = mid; else hi = mid;
    }
    int prev;
    if (req_q_start[lo] == t) {
      const int slot = state_slots[lo];
      prev = last_id[slot] - 1;
      last_id[slot] = ids[req_q_start[lo + 1] - 1] + 1;
    } else {
      prev = ids[t - 1];
    }
    prev_s = positions[t] == 0 ? -1 : prev;
  }
  __syncthreads();
  const int id = ids[t], prev = prev_s;
  float* dst = out + (size_t)t * width;
  if (id < 0 || id >= vocab || prev >= vocab) {  // refuse rather than read outside the table
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const long long hashed = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
  const T* a = table + (size_t)id * width;
  const T* b = pairs + (size_t)(prev < 0 ? buckets : (int)hashed) * width;
  if (sizeof(T) == 2 && width % 8 == 0 && (((uintptr_t)table | (uintptr_t)pairs | (uintptr_t)out) & 15) == 0) {
    // eight entries a thread: one 16-byte load from each table, two 16-byte stores
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      const uint4 ra = *reinterpret_cast<const uint4*>(a + i), rb = *reinterpret_cast<const uint4*>(b + i);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb);
      float sum[8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 fa = __bfloat1622float2(ha[u]), fb = __bfloat1622float2(hb[u]);
        sum[2 * u] = fa.x + fb.x;
        sum[2 * u + 1] = fa.y + fb.y;
      }
      *reinterpret_cast<float4*>(dst + i) = make_float4(sum[0], sum[1], sum[2], sum[3]);
      *reinterpret_cast<float4*>(dst + i + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = asb::to_float(a[i]) + asb::to_float(b[i]);
}

template <typename T>
__global__ void concat_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                   int width, long long total) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  if (width % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0) {
    // four entries a thread (no group of four straddles the two halves of a row)
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < total; i += (long long)gridDim.x * blockDim.x * 4) {
      const long long r = i / (2 * width);
      const int c = (int)(i - r * 2 * width);
      const float4 v = *reinterpret_cast<const float4*>(c < width ? a + r * width + c : b + r * width + c - width);
      if (sizeof(T) == 2) {  // one 8-byte store
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(out + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      } else {
        out[i] = asb::from_float<T>(v.x);
        out[i + 1] = asb::from_float<T>(v.y);
        out[i + 2] = asb::from_float<T>(v.z);
        out[i + 3] = asb::from_float<T>(v.w);
      }
    }
    return;
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (2 * width);
    const int c = (int)(i - r * 2 * width);
    out[i] = asb::from_float<T>(c < width ? a[r * width + c] : b[r * width + c - width]);
  }
}

}  // namespace

// out32, out1, out2, x, y1, y2, bias: each may be null (out2 with gain2). dtype is that of out1/out2.
extern "C" int asb_residual_dual_norm(float* out32, void* out1, void* out2, const float* x, const float* y1,
                                      const float* y2, const float* bias, const float* gain1, const float* gain2,
                                      int n, int width, float mult, float eps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (width < 1 || width > 48 * 1024 / 4) return asb::fail("residual_dual_norm: width %d not in 1..12288", width);
  if ((out1 && !gain1) || (out2 && !gain2)) return asb::fail("residual_dual_norm: a normed output needs its gain");
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(residual_dual_norm_kernel<T>, n, threads_for(width), width * sizeof(float),
                                           stream, out32, (T*)out1, (T*)out2, x, y1, y2, bias, gain1, gain2, width,
                                           mult, eps));
  return asb::check_launch("residual_dual_norm");
}

extern "C" int asb_pair_embedding(float* out, const void* table, const void* pairs, const int* ids,
                                  const int* positions, const int* req_q_start, const int* state_slots,
                                  int* last_id, int num_tokens, int R, int width, int vocab, int buckets,
                                  int mul_prev, int mul_cur, int dtype, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (buckets < 1 || R < 1) return asb::fail("pair_embedding: %d buckets, %d requests", buckets, R);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(pair_embedding_kernel<T>, num_tokens, threads_for(sizeof(T) == 2 && width % 8 == 0 ? width / 8 : width), 0, stream, out,
                                           (const T*)table, (const T*)pairs, ids, positions, req_q_start, state_slots,
                                           last_id, R, width, vocab, buckets, mul_prev, mul_cur, status));
  return asb::check_launch("pair_embedding");
}

extern "C" int asb_concat_cast(void* out, const float* a, const float* b, int n, int width, int dtype,
                               cudaStream_t stream) {
  if (n == 0) return 0;
  const long long total = (long long)n * 2 * width;
  const long long blocks = (total / (width % 4 == 0 ? 4 : 1) + 255) / 256;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(concat_cast_kernel<T>, (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256,
                                           0, stream, (T*)out, a, b, width, total));
  return asb::check_launch("concat_cast");
}
