// Linear attention with a fixed decay per head ("lightning attention"), as a recurrence over a
// request's tokens:
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        S: [D, V] per (request, head), float32, kept in the
//   o_t = S_t^T q_t                          request's state slot between steps
//
// q, k and v are column ranges of one projection [T, stride] in the compute dtype; `act` 1
// applies SiLU to them on the way in (float32). The state, the outer products, the decay and
// the outputs are float32.
//
// Work split: grid (request, head, chunk of value columns). A thread owns one value column and
// RPT rows of S in registers (D is covered by DS = 2^n adjacent lanes of RPT rows each, whose
// partial outputs are added by shuffles), so a token costs no block-wide synchronisation: a
// tile of TT tokens is staged in shared memory at once and walked in registers. The tokens of a
// request are walked in order whatever the step holds (a whole prompt, a portion, one decoded
// token), so the result does not depend on how a prompt was cut.
//
// Long portions are cut into segments that run side by side (the caller names them by their row
// bounds): each segment runs the recurrence from a zero state (mode 1) and leaves its own
// contribution; asb_lightning_scan walks a request's segments in order, S <- decay^n S + own,
// leaving the state each segment starts from and the request's final state in its slot; mode 2
// then adds decay^(t - first + 1) S_first^T q_t to every token of a segment. The sums are the
// recurrence's, grouped differently: equal beyond rounding.
//
// The same kernel serves the other recurrences of this form (asb_linear_recurrence):
//   - a decay and an input weight per token and head, S_t = a_t S_(t-1) + b_t k_t v_t^T, read from
//     float32 arrays [T, H] (gated matrix memories; the arrays come from the gates' own scan);
//   - a normaliser n_t = a_t n_(t-1) + b_t k_t kept beside S and n_t . q_t given out with o_t: the
//     first warp of a (request, head)'s first block walks it through shared memory ahead of its
//     share of S (a few multiply-adds a token);
//   - a rotation of q and k by position (pairs (i, i + rot / 2) of the first `rot` entries of a
//     head; the cosines and sines come from a table [T, rot / 2] made once per step by
//     asb_rotary_table, float32 `sincosf` of position * inv_freq[i]) and a scale on each, applied as
//     a tile is staged.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kTokenTile = 16;

struct LightningParams {
  float* out;               // [T, H * V]
  const void* proj;         // [T, stride]
  float* state;             // [slots, H, D, V]
  const int* state_slots;   // [R]
  const int* req_q_start;   // [R + 1]
  const float* decay;       // [H]
  int stride, q_off, k_off, v_off;
  int H, D, V, DS, act;
  int dp_shift, cpb_shift;  // log2 of the padded rows DS * RPT and of the value columns a block
  int zero_init;  // 1: the state starts at zero and is only written (a segment's local state)
  int carry;      // 1: add each token's share of the state it started from instead of running the recurrence
  const float* tok_decay;   // [T, H] a decay per token, or null: decay[h]
  const float* tok_gain;    // [T, H] a weight on each token's outer product, or null: 1
  float* norm_state;        // [slots, H, D] the normaliser, or null: none is kept
  float* norm_out;          // [T, H] n_t . q_t
  float* through;           // [R, H] with per-token decays, from-zero pass: the product of a segment's decays
  const float2* rot_table;  // [T, rot / 2] (cos, sin) of each token's angles, or null: no rotation
  int rot;
  float q_scale, k_scale;
  int qk_share;             // this many neighbouring heads read one q and one k (grouped state-space layers); 1: a q and k per head
};

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }

// GEN false: the fixed-decay form alone (per-token arrays, normaliser and rotation compiled out).
template <typename T, int RPT, bool GEN>
__global__ void __launch_bounds__(kThreads)
lightning_kernel(const LightningParams p) {
  const float* tok_decay = GEN ? p.tok_decay : nullptr;
  const float* tok_gain = GEN ? p.tok_gain : nullptr;
  float* norm_state = GEN ? p.norm_state : nullptr;
  const float2* rot_table = GEN ? p.rot_table : nullptr;
  const int hq = GEN ? (int)blockIdx.y / p.qk_share : (int)blockIdx.y;  // whose q and k columns this head reads
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  extern __shared__ float smem[];
  const int DS = p.DS, DP = DS * RPT;    // padded rows
  const int CPB = kThreads / DS;          // value columns per block
  float* qs = smem;                       // [TT][DP]
  float* ks = qs + kTokenTile * DP;       // [TT][DP]
  float* vs = ks + kTokenTile * DP;       // [TT][CPB]
  __shared__ float decs[kTokenTile], gains[kTokenTile];
  float* ns = vs + kTokenTile * CPB;      // [DP] the normaliser (general form, first block of a head)
  const int r = blockIdx.x, h = blockIdx.y;
  const int ds = threadIdx.x & (DS - 1), cl = threadIdx.x >> (7 - p.cpb_shift);  // DS and 128 / DS are powers of two
  const int col = blockIdx.z * CPB + cl;
  const int row_lo = p.req_q_start[r], row_hi = p.req_q_start[r + 1];
  const int slot = p.state_slots[r];
  const float dec = p.decay ? p.decay[h] : 1.f;
  const bool live = col < p.V;
  float* sp = p.state + (((size_t)slot * p.H + h) * p.D) * p.V + col;
  const size_t sstride = p.V;
  // the normaliser is the first warp's of the head's first block
  const bool keeps_norm = GEN && norm_state != nullptr && blockIdx.z == 0 && threadIdx.x < 32;
  float* np_ = norm_state ? norm_state + ((size_t)slot * p.H + h) * p.D : nullptr;
  if (keeps_norm)
    for (int d = threadIdx.x; d < p.D; d += 32) ns[d] = p.zero_init ? 0.f : np_[d];
  const int half = p.rot >> 1;

  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = ds * RPT + i;
    S[i] = (live && d < p.D && !p.zero_init) ? sp[(size_t)d * sstride] : 0.f;
  }
  const T* proj = (const T*)p.proj;
  float weight = 1.f;
  for (int t0 = row_lo; t0 < row_hi; t0 += kTokenTile) {
    const int nt = min(kTokenTile, row_hi - t0);
    __syncthreads();
    // the tile's loads are issued eight at a time before any is used
    constexpr int U = 8;
    if (threadIdx.x < nt) {
      decs[threadIdx.x] = tok_decay ? tok_decay[(size_t)(t0 + threadIdx.x) * p.H + h] : dec;
      gains[threadIdx.x] = tok_gain ? tok_gain[(size_t)(t0 + threadIdx.x) * p.H + h] : 1.f;
    }
    for (int base = threadIdx.x; base < nt * DP; base += kThreads * U) {
      float qv[U], kv[U], qp[U], kp[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * kThreads;
        const int t = i >> p.dp_shift, d = i - (t << p.dp_shift);
        qv[u] = kv[u] = qp[u] = kp[u] = 0.f;
        if (i < nt * DP && d < p.D) {
          const T* row = proj + (size_t)(t0 + t) * p.stride + hq * p.D + d;
          qv[u] = asb::to_float(row[p.q_off]);
          if (!p.carry) kv[u] = asb::to_float(row[p.k_off]);
          if (rot_table && d < p.rot) {  // the other entry of this one's pair
            const int other = d < half ? half : -half;
            qp[u] = asb::to_float(row[p.q_off + other]);
            if (!p.carry) kp[u] = asb::to_float(row[p.k_off + other]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + u * kThreads;
        if (i < nt * DP) {
          float qx = p.act ? silu(qv[u]) : qv[u], kx = p.act ? silu(kv[u]) : kv[u];
          const int t = i >> p.dp_shift, d = i - (t << p.dp_shift);
          if (rot_table && d < p.rot) {
            const float2 turn = rot_table[(size_t)(t0 + t) * half + (d < half ? d : d - half)];
            const float cs = turn.x, sn = turn.y;
            const float qo = p.act ? silu(qp[u]) : qp[u], ko = p.act ? silu(kp[u]) : kp[u];
            qx = d < half ? qx * cs - qo * sn : qx * cs + qo * sn;
            kx = d < half ? kx * cs - ko * sn : kx * cs + ko * sn;
          }
          qs[i] = GEN ? qx * p.q_scale : qx;
          ks[i] = GEN ? kx * p.k_scale : kx;
        }
      }
    }
    if (!p.carry) {
      for (int base = threadIdx.x; base < nt * CPB; base += kThreads * U) {
        float vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = base + u * kThreads;
          const int t = i >> p.cpb_shift, c = blockIdx.z * CPB + (i - (t << p.cpb_shift));
          vv[u] = (i < nt * CPB && c < p.V) ? asb::to_float(proj[(size_t)(t0 + t) * p.stride + p.v_off + h * p.V + c]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = base + u * kThreads;
          if (i < nt * CPB) {
            const float v = p.act ? silu(vv[u]) : vv[u];
            vs[i] = tok_gain ? v * tok_gain[(size_t)(t0 + (i >> p.cpb_shift)) * p.H + h] : v;
          }
        }
      }
    }
    __syncthreads();
    if (keeps_norm) {
      // n_t = a_t n_(t-1) + b_t k_t and n_t . q_t, or in the carried pass the share of the n this segment started from
      // (a lane owns rows d = lane, lane + 32, ...: the tile's tokens are walked row by row, and the
      // sixteen sums over the lanes are formed together afterwards, their shuffles in flight at once)
      float part[kTokenTile];
#pragma unroll
      for (int t = 0; t < kTokenTile; ++t) part[t] = 0.f;
      const float n_so_far = (p.carry && (int)threadIdx.x < nt) ? p.norm_out[(size_t)(t0 + threadIdx.x) * p.H + h] : 0.f;
      for (int d = threadIdx.x; d < p.D; d += 32) {
        float n = ns[d];
#pragma unroll
        for (int t = 0; t < kTokenTile; ++t) {
          if (t < nt) {
            if (!p.carry) n = fmaf(decs[t], n, gains[t] * ks[t * DP + d]);
            part[t] = fmaf(n, qs[t * DP + d], part[t]);
          }
        }
        ns[d] = n;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int t = 0; t < kTokenTile; ++t) part[t] += __shfl_xor_sync(0xffffffffu, part[t], off);
      float w = weight;
#pragma unroll
      for (int t = 0; t < kTokenTile; ++t) {
        w *= t < nt ? decs[t] : 1.f;
        if (threadIdx.x == t && t < nt) {
          p.norm_out[(size_t)(t0 + t) * p.H + h] = p.carry ? fmaf(w, part[t], n_so_far) : part[t];
        }
      }
    }
    if (p.carry) {
      // o_t += decay^(t - first + 1) * S_first^T q_t: what the tokens before this segment contribute
      // (the tile's outputs so far are fetched together first, so that no token waits for its own)
      float so_far[kTokenTile];
#pragma unroll
      for (int t = 0; t < kTokenTile; ++t)
        so_far[t] = (ds == 0 && live && t < nt) ? p.out[(size_t)(t0 + t) * p.H * p.V + h * p.V + col] : 0.f;
#pragma unroll
      for (int t = 0; t < kTokenTile; ++t) {
        if (t >= nt) break;
        const float4* qr = reinterpret_cast<const float4*>(qs + t * DP + ds * RPT);
        float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < RPT; i += 4) {
          const float4 qq = qr[i >> 2];
          o4[0] = fmaf(S[i], qq.x, o4[0]);
          o4[1] = fmaf(S[i + 1], qq.y, o4[1]);
          o4[2] = fmaf(S[i + 2], qq.z, o4[2]);
          o4[3] = fmaf(S[i + 3], qq.w, o4[3]);
        }
        float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        for (int off = 1; off < DS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        weight *= decs[t];
        if (ds == 0 && live) p.out[(size_t)(t0 + t) * p.H * p.V + h * p.V + col] = fmaf(weight, o, so_far[t]);
      }
      continue;
    }
    if (GEN && p.through && p.zero_init && blockIdx.z == 0 && threadIdx.x == 32 % kThreads)
      for (int t = 0; t < nt; ++t) weight *= decs[t];  // (weight is otherwise the carried pass's)
    for (int t = 0; t < nt; ++t) {
      const float vv = vs[t * CPB + cl], dec = decs[t];
      const float4* kr = reinterpret_cast<const float4*>(ks + t * DP + ds * RPT);
      const float4* qr = reinterpret_cast<const float4*>(qs + t * DP + ds * RPT);
      float o4[4] = {0.f, 0.f, 0.f, 0.f};  // four chains instead of one of RPT dependent additions
#pragma unroll
      for (int i = 0; i < RPT; i += 4) {
        const float4 kk = kr[i >> 2], qq = qr[i >> 2];
        S[i] = fmaf(dec, S[i], kk.x * vv);
        S[i + 1] = fmaf(dec, S[i + 1], kk.y * vv);
        S[i + 2] = fmaf(dec, S[i + 2], kk.z * vv);
        S[i + 3] = fmaf(dec, S[i + 3], kk.w * vv);
        o4[0] = fmaf(S[i], qq.x, o4[0]);
        o4[1] = fmaf(S[i + 1], qq.y, o4[1]);
        o4[2] = fmaf(S[i + 2], qq.z, o4[2]);
        o4[3] = fmaf(S[i + 3], qq.w, o4[3]);
      }
      float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
      for (int off = 1; off < DS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (ds == 0 && live) p.out[(size_t)(t0 + t) * p.H * p.V + h * p.V + col] = o;
    }
  }
  if (p.carry) return;
  if (GEN && p.through && p.zero_init && blockIdx.z == 0 && threadIdx.x == 32 % kThreads) p.through[(size_t)r * p.H + h] = weight;
  if (keeps_norm)
    for (int d = threadIdx.x; d < p.D; d += 32) np_[d] = ns[d];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = ds * RPT + i;
    if (live && d < p.D) sp[(size_t)d * sstride] = S[i];
  }
}

template <typename T, int RPT>
int launch(const LightningParams& p, int R, cudaStream_t stream) {
  const int CPB = kThreads / p.DS;
  const size_t smem = sizeof(float) * (kTokenTile * (2 * p.DS * RPT + CPB) + p.DS * RPT);
  const bool general = p.tok_decay || p.tok_gain || p.norm_state || p.rot_table || p.q_scale != 1.f || p.k_scale != 1.f || p.qk_share != 1;
  auto kern = general ? lightning_kernel<T, RPT, true> : lightning_kernel<T, RPT, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return asb::fail("lightning_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
  dim3 grid(R, p.H, (p.V + CPB - 1) / CPB);
  asb::launch(kern, grid, kThreads, smem, stream, p);
  return asb::check_launch("lightning_attention");
}

// Between the segments of a request: the state each segment starts from, and the request's state
// after its last one. local[c] holds segment c's own contribution on entry and the state the
// segment starts from on exit; an element per thread, the segments of a request in order.
__global__ void lightning_scan_kernel(float* __restrict__ local, float* __restrict__ state,
                                      const int* __restrict__ state_slots, const int* __restrict__ req_seg_start,
                                      const int* __restrict__ seg_bounds, const float* __restrict__ decay,
                                      const float* __restrict__ seg_through, int H, int DV) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y;
  const float dec = decay ? decay[h] : 1.f, log_dec = logf(dec);
  float* sp = state + ((size_t)state_slots[r] * H + h) * DV;
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < DV; e += gridDim.z * blockDim.x) {
    float S = sp[e];
    const int c_end = req_seg_start[r + 1];
    for (int c0 = req_seg_start[r]; c0 < c_end; c0 += 8) {
      // eight segments' contributions are fetched before the chain through them is walked
      float own[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) own[u] = c0 + u < c_end ? local[((size_t)(c0 + u) * H + h) * DV + e] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u;
        if (c >= c_end) break;
        local[((size_t)c * H + h) * DV + e] = S;
        float through;  // what is left of a state after the segment's tokens
        if (seg_through) {
          through = seg_through[(size_t)c * H + h];
        } else {
          const float n = (float)(seg_bounds[c + 1] - seg_bounds[c]);
          through = dec == 1.f ? 1.f : expf(n * log_dec);
        }
        S = fmaf(through, S, own[u]);
      }
    }
    sp[e] = S;
  }
}

// (cos, sin) of position * inv_freq[i] for every token of a step, float32: once per step for all
// the layers that rotate by the same frequencies.
__global__ void rotary_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int half, long long total) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float sn, cs;
    sincosf((float)positions[i / half] * inv_freq[i % half], &sn, &cs);
    table[i] = make_float2(cs, sn);
  }
}

}  // namespace

extern "C" int asb_rotary_table(float* table, const int* positions, const float* inv_freq, int num_tokens, int half,
                                cudaStream_t stream) {
  if (num_tokens == 0 || half == 0) return 0;
  const long long total = (long long)num_tokens * half;
  const long long blocks = (total + 255) / 256;
  asb::launch(rotary_table_kernel, (unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream,
              reinterpret_cast<float2*>(table), positions, inv_freq, half, total);
  return asb::check_launch("rotary_table");
}

// D * V elements per (request, head); for a normaliser, call it with its own buffers and V = 1.
// seg_through [segments, H]: what is left of a state after each segment (the from-zero pass of
// asb_linear_recurrence writes it when the decays are per token), or null: decay[h]^tokens.
extern "C" int asb_recurrence_scan(float* local, float* state, const int* state_slots, const int* req_seg_start,
                                   const int* seg_bounds, const float* decay, const float* seg_through, int R, int H,
                                   int D, int V, cudaStream_t stream) {
  if (R == 0) return 0;
  if (!decay && !seg_through) return asb::fail("recurrence_scan: no decay given");
  const int DV = D * V;
  dim3 grid(R, H, (DV + 255) / 256 < 64 ? (DV + 255) / 256 : 64);
  asb::launch(lightning_scan_kernel, grid, 256, 0, stream, local, state, state_slots, req_seg_start, seg_bounds, decay,
              seg_through, H, DV);
  return asb::check_launch("recurrence_scan");
}

extern "C" int asb_lightning_scan(float* local, float* state, const int* state_slots, const int* req_seg_start,
                                  const int* seg_bounds, const float* decay, int R, int H, int D, int V,
                                  cudaStream_t stream) {
  return asb_recurrence_scan(local, state, state_slots, req_seg_start, seg_bounds, decay, nullptr, R, H, D, V, stream);
}

// The general form. decay [H] or tok_decay [T, H] (one of them); tok_gain [T, H] or null;
// norm_state [slots, H, D] with norm_out [T, H], or both null; rot_table [T, rot / 2, 2] (asb_rotary_table), or null.
// qk_share: every group of this many neighbouring heads shares one q and one k (H / qk_share heads
// of D columns from q_off and k_off); the values, states and outputs stay per head.
extern "C" int asb_linear_recurrence_shared(float* out, const void* proj, int stride, int q_off, int k_off, int v_off,
                                            float* state, const int* state_slots, const int* req_q_start,
                                            const float* decay, const float* tok_decay, const float* tok_gain,
                                            float* norm_state, float* norm_out, float* through, const float* rot_table,
                                            int rot, float q_scale, float k_scale, int R, int H, int D, int V, int act,
                                            int mode, int qk_share, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  if (qk_share < 1 || H % qk_share) return asb::fail("linear_recurrence: %d heads do not share q and k in groups of %d", H, qk_share);
  if (H < 1 || D < 1 || V < 1 || H > 65535) return asb::fail("linear_recurrence: %d heads of %d x %d", H, D, V);
  if (!decay && !tok_decay) return asb::fail("linear_recurrence: no decay given");
  if ((norm_state == nullptr) != (norm_out == nullptr)) return asb::fail("linear_recurrence: a normaliser needs its state and its output");
  if (rot_table && (rot < 0 || rot % 2 || rot > D)) return asb::fail("linear_recurrence: rotation of %d of %d entries", rot, D);
  LightningParams p;
  p.out = out; p.proj = proj; p.state = state; p.state_slots = state_slots; p.req_q_start = req_q_start;
  p.decay = decay; p.stride = stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.H = H; p.D = D; p.V = V; p.act = act;
  p.tok_decay = tok_decay; p.tok_gain = tok_gain; p.norm_state = norm_state; p.norm_out = norm_out;
  p.through = (mode == 1 && tok_decay) ? through : nullptr;
  p.rot_table = (rot_table && rot > 0) ? reinterpret_cast<const float2*>(rot_table) : nullptr; p.rot = rot;
  p.q_scale = q_scale; p.k_scale = k_scale; p.qk_share = qk_share;
  p.zero_init = mode == 1;  // mode 0: the recurrence from the slots' states; 1: from zero, per segment; 2: the carried share
  p.carry = mode == 2;
  // rows of the state per thread: 64 from D = 64 on, fewer for narrow heads; D beyond 64 is
  // shared among 2, 4, ... lanes (32 rows a thread at D = 128 measured slower: 1.23 against 0.76 ms
  // for 2,048 tokens of 16 heads)
  const int rpt = D >= 64 ? 64 : (D > 16 ? 32 : 16);
  int ds = 1;
  while (ds * rpt < D) ds <<= 1;
  if (ds > 32) return asb::fail("lightning_attention: key size %d exceeds %d", D, 32 * 64);
  p.DS = ds;
  p.dp_shift = 0;
  while ((1 << p.dp_shift) < ds * rpt) ++p.dp_shift;
  p.cpb_shift = 0;
  while ((1 << p.cpb_shift) < kThreads / ds) ++p.cpb_shift;
  if ((V + kThreads / ds) / (kThreads / ds) > 65535) return asb::fail("linear_recurrence: value size %d", V);
  ASB_DISPATCH_DTYPE(dtype, T, {
    if (rpt == 64) return launch<T, 64>(p, R, stream);
    if (rpt == 32) return launch<T, 32>(p, R, stream);
    return launch<T, 16>(p, R, stream);
  });
  return 0;
}

extern "C" int asb_linear_recurrence(float* out, const void* proj, int stride, int q_off, int k_off, int v_off,
                                     float* state, const int* state_slots, const int* req_q_start,
                                     const float* decay, const float* tok_decay, const float* tok_gain,
                                     float* norm_state, float* norm_out, float* through, const float* rot_table,
                                     int rot, float q_scale, float k_scale, int R, int H, int D, int V, int act,
                                     int mode, int dtype, cudaStream_t stream) {
  return asb_linear_recurrence_shared(out, proj, stride, q_off, k_off, v_off, state, state_slots, req_q_start, decay,
                                      tok_decay, tok_gain, norm_state, norm_out, through, rot_table, rot, q_scale, k_scale,
                                      R, H, D, V, act, mode, 1, dtype, stream);
}

extern "C" int asb_lightning_attention(float* out, const void* proj, int stride, int q_off, int k_off, int v_off,
                                       float* state, const int* state_slots, const int* req_q_start,
                                       const float* decay, int R, int H, int D, int V, int act, int mode, int dtype,
                                       cudaStream_t stream) {
  return asb_linear_recurrence(out, proj, stride, q_off, k_off, v_off, state, state_slots, req_q_start, decay, nullptr,
                               nullptr, nullptr, nullptr, nullptr, nullptr, 0, 1.f, 1.f, R, H, D, V, act, mode, dtype, stream);
}
