// A gated linear unit on a (gate, up) pair of float32 sums: act(gate + b_gate) * (up + b_up), with
// act the SiLU, the tanh form of GELU or the exact GELU. The tensor-core GEMMs apply it in their
// epilogues to products whose weight rows alternate gate_i, up_i (row n the gate, row n + 1 the up
// of output column n / 2); `bias`, float32 in the same alternating order, may be null.
#pragma once

namespace asb {

enum GluAct : int { kGluSilu = 0, kGluGeluTanh = 1, kGluGelu = 2 };

template <int ACT>
__device__ __forceinline__ float glu_value(float gate, float up) {
  if (ACT == kGluSilu) return gate / (1.f + __expf(-gate)) * up;
  if (ACT == kGluGeluTanh) {
    // 0.5 g (1 + tanh(u)) = g / (1 + exp(-2u)), u = sqrt(2 / pi) (g + 0.044715 g^3): one fast exponential, as
    // the SiLU's; its error (a few float32 steps) is far below the rounding to bfloat16 that follows
    const float u2 = 1.59576912160573072f * fmaf(0.044715f * gate * gate, gate, gate);
    return gate / (1.f + __expf(-u2)) * up;
  }
  return 0.5f * gate * (1.f + erff(gate * 0.70710678118654752f)) * up;
}

__device__ __forceinline__ float glu_pair(float gate, float up, const float* __restrict__ bias, int n, int act) {
  if (bias) {
    gate += bias[n];
    up += bias[n + 1];
  }
  if (act == kGluSilu) return glu_value<kGluSilu>(gate, up);
  if (act == kGluGeluTanh) return glu_value<kGluGeluTanh>(gate, up);
  return glu_value<kGluGelu>(gate, up);
}

// N float32 sums of one token over N neighbouring weight rows (gate, up, gate, ...; biases already added) to
// N / 2 gated values in bfloat16: the activation is chosen once, outside the loop over the pairs.
template <int N>
__device__ __forceinline__ void glu_pairs(const uint32_t (&raw)[N], __nv_bfloat16* out, int act) {
  if (act == kGluSilu) {
#pragma unroll
    for (int j = 0; j < N / 2; ++j) out[j] = __float2bfloat16_rn(glu_value<kGluSilu>(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1])));
  } else if (act == kGluGeluTanh) {
#pragma unroll
    for (int j = 0; j < N / 2; ++j) out[j] = __float2bfloat16_rn(glu_value<kGluGeluTanh>(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1])));
  } else {
#pragma unroll
    for (int j = 0; j < N / 2; ++j) out[j] = __float2bfloat16_rn(glu_value<kGluGelu>(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1])));
  }
}

// Adds bias[n], ..., bias[n + N - 1] to N float32 sums that a thread holds as raw bits (one token's sums over N
// neighbouring weight rows), the first `valid` of them: with all N and a 16-byte aligned start as N / 4 loads of
// four floats, issued together (every lane of a warp reads the same addresses), else one by one.
template <int N>
__device__ __forceinline__ void add_bias(uint32_t (&raw)[N], const float* __restrict__ bias, int n, int valid) {
  const float* b = bias + n;
  if (valid >= N && (((uintptr_t)b) & 15) == 0) {
    float4 v[N / 4];
#pragma unroll
    for (int j = 0; j < N / 4; ++j) v[j] = __ldg(reinterpret_cast<const float4*>(b) + j);
#pragma unroll
    for (int j = 0; j < N / 4; ++j) {
      raw[4 * j] = __float_as_uint(__uint_as_float(raw[4 * j]) + v[j].x);
      raw[4 * j + 1] = __float_as_uint(__uint_as_float(raw[4 * j + 1]) + v[j].y);
      raw[4 * j + 2] = __float_as_uint(__uint_as_float(raw[4 * j + 2]) + v[j].z);
      raw[4 * j + 3] = __float_as_uint(__uint_as_float(raw[4 * j + 3]) + v[j].w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j < valid) raw[j] = __float_as_uint(__uint_as_float(raw[j]) + __ldg(b + j));
  }
}

}  // namespace asb
