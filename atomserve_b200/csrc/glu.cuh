// A gated linear unit on a (gate, up) pair of float32 sums: act(gate + b_gate) * (up + b_up), with
// act the SiLU, the tanh form of GELU or the exact GELU. The tensor-core GEMMs apply it in their
// epilogues to products whose weight rows alternate gate_i, up_i (row n the gate, row n + 1 the up
// of output column n / 2); `bias`, float32 in the same alternating order, may be null.
#pragma once

namespace asb {

enum GluAct : int { kGluSilu = 0, kGluGeluTanh = 1, kGluGelu = 2 };

__device__ __forceinline__ float glu_pair(float gate, float up, const float* __restrict__ bias, int n, int act) {
  if (bias) {
    gate += bias[n];
    up += bias[n + 1];
  }
  if (act == kGluSilu) return gate / (1.f + __expf(-gate)) * up;
  if (act == kGluGeluTanh) return 0.5f * gate * (1.f + tanhf(0.79788456080286536f * (gate + 0.044715f * gate * gate * gate))) * up;
  return 0.5f * gate * (1.f + erff(gate * 0.70710678118654752f)) * up;
}

}  // namespace asb
