// Kernels for blocks that norm a sublayer's input and its output, x <- x + N_out(f(N_in(x))), over a
// float32 residual stream, N the RMS norm v / sqrt(mean(v^2) + eps) times a gain. Everything inside
// is float32; each stored value is rounded once.
//
//   asb_add_normed          s = x + N_out(y + bias) (bias optional), written as float32; and, where a
//                           second gain is given, N_next(s) in the compute dtype: what the next
//                           sublayer's products read. One block per row, the row kept in shared memory.
//   asb_partial_add_normed  the same with y given as the partial sums that the tensor-core GEMM left
//                           in its workspace (few tokens): a thread adds up the slots of 8 columns
//                           itself, in the order of the GEMM's own reduction.
//   asb_bias_glu            act(gate + b_gate) * (up + b_up) of a stacked product [T, 2F] (gate
//                           columns first); act: SiLU, the tanh form of GELU, or the exact GELU.
//   asb_softcap             v <- cap tanh(v / cap) in place, float32 (an output head's logits).
#include "common.cuh"
#include "gemm_partials.cuh"

namespace {

template <typename TY, typename T>
__global__ void add_normed_kernel(float* __restrict__ out32, T* __restrict__ out_c, const float* __restrict__ x,
                                  const TY* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ gain_out,
                                  const float* __restrict__ gain_next, int width, float eps_out, float eps_next) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const size_t at = (size_t)blockIdx.x * width;
  const float inv_w = 1.f / (float)width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = asb::to_float(y[at + i]);
    if (bias) v += bias[i];
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) * inv_w + eps_out);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {  // (each thread reads back what it wrote)
    const float s = fmaf(row[i] * inv, gain_out[i], x[at + i]);
    row[i] = s;
    out32[at + i] = s;
    s2 = fmaf(s, s, s2);
  }
  if (!gain_next) return;
  const float inv2 = 1.f / sqrtf(asb::block_sum(s2, scratch) * inv_w + eps_next);
  for (int i = threadIdx.x; i < width; i += blockDim.x) out_c[at + i] = asb::from_float<T>(row[i] * inv2 * gain_next[i]);
}

__global__ void partial_add_normed_kernel(float* __restrict__ out32, __nv_bfloat16* __restrict__ out_c,
                                          const asb::PartialSums ps, const float* __restrict__ x,
                                          const float* __restrict__ bias, const float* __restrict__ gain_out,
                                          const float* __restrict__ gain_next, int width, float eps_out, float eps_next) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, i = threadIdx.x * 8;
  const bool active = i < width;
  const int slots = active ? asb::partial_slots(ps, i / asb::kPartialRows) : 0;
  float g[8], gn[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    g[k] = active ? gain_out[i + k] : 0.f;
    gn[k] = (active && gain_next) ? gain_next[i + k] : 0.f;
    b[k] = (active && bias) ? bias[i + k] : 0.f;
  }
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  float y[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) y[k] = 0.f;
  if (active) asb::partial_sum<8>(ps, t, i, slots, y);
  const float inv_w = 1.f / (float)width;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    y[k] += b[k];
    ss = fmaf(y[k], y[k], ss);
  }
  const float inv = 1.f / sqrtf(asb::block_sum(ss, scratch) * inv_w + eps_out);
  float s[8], s2 = 0.f;
  if (active) {
    const float4 x0 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i);
    const float4 x1 = *reinterpret_cast<const float4*>(x + (size_t)t * width + i + 4);
    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      s[k] = fmaf(y[k] * inv, g[k], xs[k]);
      s2 = fmaf(s[k], s[k], s2);
    }
    *reinterpret_cast<float4*>(out32 + (size_t)t * width + i) = make_float4(s[0], s[1], s[2], s[3]);
    *reinterpret_cast<float4*>(out32 + (size_t)t * width + i + 4) = make_float4(s[4], s[5], s[6], s[7]);
  }
  if (!gain_next) return;
  const float inv2 = 1.f / sqrtf(asb::block_sum(s2, scratch) * inv_w + eps_next);
  if (!active) return;
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16_rn(s[k] * inv2 * gn[k]);
  *reinterpret_cast<uint4*>(out_c + (size_t)t * width + i) = packed;
}

__device__ __forceinline__ float act_f(float z, int kind) {
  if (kind == 0) return z / (1.f + expf(-z));
  if (kind == 1) return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
  return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
}

template <typename T>
__global__ void bias_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, const float* __restrict__ bias, int inter,
                                long long total, int kind) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    float g = asb::to_float(gu[t * 2 * inter + i]), u = asb::to_float(gu[t * 2 * inter + inter + i]);
    if (bias) {
      g += bias[i];
      u += bias[inter + i];
    }
    out[idx] = asb::from_float<T>(act_f(g, kind) * u);
  }
}

__global__ void softcap_kernel(float* __restrict__ v, long long total, float cap) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const float inv = 1.f / cap;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}

unsigned grid_for(long long total) {
  const long long blocks = (total + 255) / 256;
  return (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
}

}  // namespace

// x, out32: float32 [n, width]; y: float32 (y_dtype 0) or bfloat16 (1) [n, width]; bias, gain_next
// may be null; out_c in `dtype` (ignored without gain_next).
extern "C" int asb_add_normed(float* out32, void* out_c, const float* x, const void* y, int y_dtype, const float* bias,
                              const float* gain_out, const float* gain_next, int n, int width, float eps_out, float eps_next,
                              int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const size_t smem = sizeof(float) * width;
  if (smem > 200 * 1024) return asb::fail("add_normed: width %d", width);
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define ASB_AN(TY, T)                                                                                                \
  {                                                                                                                  \
    auto kern = add_normed_kernel<TY, T>;                                                                            \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
    if (e != cudaSuccess) return asb::fail("add_normed: shared memory %zu: %s", smem, cudaGetErrorString(e));        \
    asb::launch(kern, n, threads, smem, stream, out32, (T*)out_c, x, (const TY*)y, bias, gain_out, gain_next, width, \
                eps_out, eps_next);                                                                                  \
  }
  ASB_DISPATCH_DTYPE(dtype, T, {
    if (y_dtype == asb::kFloat32) ASB_AN(float, T)
    else ASB_AN(__nv_bfloat16, T)
  });
#undef ASB_AN
  return asb::check_launch("add_normed");
}

extern "C" int asb_partial_add_normed(float* out32, void* out_c, const float* ws, int max_slots, int bn, int kb_per_tile,
                                      int num_tiles, int blocks, const float* x, const float* bias, const float* gain_out,
                                      const float* gain_next, int n, int width, float eps_out, float eps_next,
                                      cudaStream_t stream) {
  if (n == 0) return 0;
  if (width % 8 || width > 8192) return asb::fail("partial_add_normed: width %d", width);
  asb::PartialSums ps{ws, max_slots, bn, kb_per_tile, num_tiles, blocks};
  const int threads = ((width / 8 + 31) / 32) * 32;
  asb::launch(partial_add_normed_kernel, n, threads, 0, stream, out32, (__nv_bfloat16*)out_c, ps, x, bias, gain_out, gain_next,
              width, eps_out, eps_next);
  return asb::check_launch("partial_add_normed");
}

// kind 0: SiLU, 1: the tanh form of GELU, 2: the exact GELU. bias float32 [2 * inter] or null.
extern "C" int asb_bias_glu(void* out, const void* gate_up, const float* bias, int num_tokens, int inter, int kind, int dtype,
                            cudaStream_t stream) {
  if (num_tokens == 0 || inter == 0) return 0;
  if (kind < 0 || kind > 2) return asb::fail("bias_glu: activation %d", kind);
  const long long total = (long long)num_tokens * inter;
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(bias_glu_kernel<T>, grid_for(total), 256, 0, stream, (T*)out, (const T*)gate_up,
                                           bias, inter, total, kind));
  return asb::check_launch("bias_glu");
}

extern "C" int asb_softcap(float* values, long long total, float cap, cudaStream_t stream) {
  if (total == 0) return 0;
  if (!(cap > 0.f)) return asb::fail("softcap: cap %f", cap);
  asb::launch(softcap_kernel, grid_for(total), 256, 0, stream, values, total, cap);
  return asb::check_launch("softcap");
}
