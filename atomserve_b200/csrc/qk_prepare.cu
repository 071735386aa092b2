// What happens between an attention layer's stacked projection and its attention kernel, for
// layers whose heads hold several score maps, and what joins the maps afterwards:
//
//   asb_qk_prepare_store     from one row [H][maps][dim] q, [KV][maps][dim] k, [KV][vdim] v of the
//                            projection: rotate the first `rotary_dim` entries of every map of q and
//                            k (pair i with i + rotary_dim / 2, angle position * inv_freq[i]), scale
//                            q by 1 + coef ln(floor((position + 1) / every) + 1), and write
//                              queries [T, H * maps, hd]: map j of head h is query head h * maps + j,
//                                its `dim` entries at offset j * dim and zeros elsewhere,
//                              keys to their page as [KV, hd]: a head's maps side by side, then zeros,
//                              values to their page as [KV, hd]: vdim entries, then zeros,
//                            with hd >= max(maps * dim, vdim). A query head's product with the key
//                            head of its group is then its own map's score, so the paged attention
//                            kernels serve every map as one more query head of the group, over one
//                            copy of the values.
//   asb_differential_combine o = a1 - lambda a2 of the two maps' outputs per head, divided by its
//                            root mean square over vdim and multiplied by `post`
//
// Angles, sines, the logarithm, the difference and the norm are float32; each stored value is
// rounded once.
#include "common.cuh"

namespace {

struct PrepareParams {
  const void* proj;  // [T, row]
  void* q_out;       // [T, H * maps, hd]
  void* k_cache;     // [num_blocks, KV, bs, hd] or null
  void* v_cache;
  const int* positions;  // [T]
  const int* slots;      // [T] page * bs + offset, -1: store nothing
  const float* inv_freq;  // [rotary_dim / 2] or null
  int H, KV, maps, dim, vdim, hd, rotary_dim, bs, row;
  float temp_coef;
  int temp_every;  // 0: no query factor
};

// entry e of a map (of q or k) after the rotation; `cs` holds the token's cosines, then its sines
template <typename T>
__device__ __forceinline__ float turned(const T* map, int e, int rotary_dim, const float* cs) {
  const float v = asb::to_float(map[e]);
  if (e >= rotary_dim) return v;
  const int half = rotary_dim >> 1;
  const int i = e < half ? e : e - half;
  const float c = cs[i], s = cs[half + i];
  const float w = asb::to_float(map[e < half ? e + half : e - half]);
  return e < half ? v * c - w * s : v * c + w * s;
}

// the token's cosines and sines (float32 `sincosf` of position x frequency), once per block
__device__ __forceinline__ void fill_angles(float* cs, const PrepareParams& p, float position) {
  const int half = p.rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(position * p.inv_freq[i], &cs[half + i], &cs[i]);
  __syncthreads();
}

__device__ __forceinline__ float query_factor(const PrepareParams& p, int pos) {
  return p.temp_every > 0 ? 1.f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.f) : 1.f;
}

// The general form: one element a thread at a time, any sizes, both element types.
template <typename T>
__global__ void qk_prepare_store_kernel(const PrepareParams p) {
  extern __shared__ float cs[];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* src = (const T*)p.proj + (size_t)t * p.row;
  const int pos = p.positions[t];
  fill_angles(cs, p, (float)pos);
  const float factor = query_factor(p, pos);
  const int live = p.maps * p.dim;
  // queries
  T* q = (T*)p.q_out + (size_t)t * p.H * p.maps * p.hd;
  for (int i = threadIdx.x; i < p.H * p.maps * p.hd; i += blockDim.x) {
    const int head = i / p.hd, e = i - head * p.hd;  // head = h * maps + j
    const int j = head % p.maps;
    float v = 0.f;
    if (e >= j * p.dim && e < (j + 1) * p.dim)
      v = turned(src + (size_t)head * p.dim, e - j * p.dim, p.rotary_dim, cs) * factor;
    q[i] = asb::from_float<T>(v);
  }
  const int slot = p.slots ? p.slots[t] : -1;
  if (slot < 0 || !p.k_cache) return;
  const int page = slot / p.bs, off = slot - page * p.bs;
  const T* k = src + (size_t)p.H * live;
  const T* v = k + (size_t)p.KV * live;
  for (int i = threadIdx.x; i < p.KV * p.hd; i += blockDim.x) {
    const int g = i / p.hd, e = i - g * p.hd;
    const size_t at = (((size_t)page * p.KV + g) * p.bs + off) * p.hd + e;
    float kv = 0.f;
    if (e < live) {
      const int j = e / p.dim;
      kv = turned(k + (size_t)g * live + j * p.dim, e - j * p.dim, p.rotary_dim, cs);
    }
    ((T*)p.k_cache)[at] = asb::from_float<T>(kv);
    ((T*)p.v_cache)[at] = e < p.vdim ? v[(size_t)g * p.vdim + e] : asb::from_float<T>(0.f);
  }
}

// The vector form (bfloat16): eight entries a thread by 16-byte loads and stores, where map, value and
// head sizes and half the rotated entries are multiples of 8 (so no vector straddles a map's end or
// the two halves of a rotation) and rows and pages start on 16-byte boundaries.
struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* at) {
  const uint4 raw = *reinterpret_cast<const uint4*>(at);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  Vec8 out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out.v[2 * i] = f.x;
    out.v[2 * i + 1] = f.y;
  }
  return out;
}

__device__ __forceinline__ void store8(__nv_bfloat16* at, const Vec8& x) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x.v[2 * i], x.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(at) = raw;
}

// entries e .. e + 7 of a map after the rotation
__device__ __forceinline__ Vec8 turned8(const __nv_bfloat16* map, int e, int rotary_dim, const float* cs) {
  Vec8 v = load8(map + e);
  if (e >= rotary_dim) return v;
  const int half = rotary_dim >> 1;
  const bool low = e < half;
  const int i = low ? e : e - half;
  const Vec8 w = load8(map + (low ? e + half : e - half));
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const float c = cs[i + u], s = cs[half + i + u];
    v.v[u] = low ? v.v[u] * c - w.v[u] * s : v.v[u] * c + w.v[u] * s;
  }
  return v;
}

__global__ void qk_prepare_store_vec_kernel(const PrepareParams p) {
  extern __shared__ float cs[];
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  using T = __nv_bfloat16;
  const int t = blockIdx.x;
  const T* src = (const T*)p.proj + (size_t)t * p.row;
  const int pos = p.positions[t];
  fill_angles(cs, p, (float)pos);
  const float factor = query_factor(p, pos);
  const int live = p.maps * p.dim, per = p.hd >> 3;  // vectors a head
  Vec8 zero;
#pragma unroll
  for (int u = 0; u < 8; ++u) zero.v[u] = 0.f;
  T* q = (T*)p.q_out + (size_t)t * p.H * p.maps * p.hd;
  for (int i = threadIdx.x; i < p.H * p.maps * per; i += blockDim.x) {
    const int head = i / per, e = (i - head * per) << 3;
    const int j = head % p.maps;
    Vec8 v = zero;
    if (e >= j * p.dim && e < (j + 1) * p.dim) {
      v = turned8(src + (size_t)head * p.dim, e - j * p.dim, p.rotary_dim, cs);
#pragma unroll
      for (int u = 0; u < 8; ++u) v.v[u] *= factor;
    }
    store8(q + (size_t)head * p.hd + e, v);
  }
  const int slot = p.slots ? p.slots[t] : -1;
  if (slot < 0 || !p.k_cache) return;
  const int page = slot / p.bs, off = slot - page * p.bs;
  const T* k = src + (size_t)p.H * live;
  const T* v = k + (size_t)p.KV * live;
  for (int i = threadIdx.x; i < p.KV * per; i += blockDim.x) {
    const int g = i / per, e = (i - g * per) << 3;
    const size_t at = (((size_t)page * p.KV + g) * p.bs + off) * p.hd + e;
    Vec8 kv = zero;
    if (e < live) {
      const int j = e / p.dim;
      kv = turned8(k + (size_t)g * live + j * p.dim, e - j * p.dim, p.rotary_dim, cs);
    }
    store8((T*)p.k_cache + at, kv);
    if (e < p.vdim) *reinterpret_cast<uint4*>((T*)p.v_cache + at) = *reinterpret_cast<const uint4*>(v + (size_t)g * p.vdim + e);
    else store8((T*)p.v_cache + at, zero);
  }
}

// One warp per (token, head): a [T, H, 2, hd] -> out [T, H, vdim].
template <typename T>
__global__ void differential_combine_kernel(T* __restrict__ out, const T* __restrict__ a, int rows, int hd, int vdim,
                                            float lambda, float post, float eps) {
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* a1 = a + (size_t)row * 2 * hd;
  const T* a2 = a1 + hd;
  float ss = 0.f;
  for (int e = lane; e < vdim; e += 32) {
    const float o = fmaf(-lambda, asb::to_float(a2[e]), asb::to_float(a1[e]));
    ss = fmaf(o, o, ss);
  }
  const float inv = post / sqrtf(asb::warp_sum(ss) / (float)vdim + eps);
  for (int e = lane; e < vdim; e += 32) {
    const float o = fmaf(-lambda, asb::to_float(a2[e]), asb::to_float(a1[e]));
    out[(size_t)row * vdim + e] = asb::from_float<T>(o * inv);
  }
}

}  // namespace

extern "C" int asb_qk_prepare_store(const void* proj, void* q_out, void* k_cache, void* v_cache,
                                    const int* positions, const int* slots, const float* inv_freq, int T_,
                                    int row, int H, int KV, int maps, int dim, int vdim, int hd, int rotary_dim, int bs,
                                    float temp_coef, int temp_every, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  if (maps < 1 || dim < 1 || maps * dim > hd || vdim > hd) return asb::fail("qk_prepare_store: %d maps of %d and values of %d do not fit heads of %d", maps, dim, vdim, hd);
  if (rotary_dim % 2 || rotary_dim > dim || (rotary_dim && !inv_freq)) return asb::fail("qk_prepare_store: rotary_dim %d against dim %d", rotary_dim, dim);
  if (row < H * maps * dim + (k_cache ? KV * (maps * dim + vdim) : 0)) return asb::fail("qk_prepare_store: rows of %d hold no such projection", row);
  if (k_cache && (!v_cache || !slots || bs < 1)) return asb::fail("qk_prepare_store: pages need values, slots and a page size");
  PrepareParams p;
  p.proj = proj; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.slots = slots; p.inv_freq = inv_freq;
  p.H = H; p.KV = KV; p.maps = maps; p.dim = dim; p.vdim = vdim; p.hd = hd; p.rotary_dim = rotary_dim; p.bs = bs;
  p.row = row;
  p.temp_coef = temp_coef; p.temp_every = temp_every;
  const size_t smem = sizeof(float) * (size_t)(rotary_dim > 0 ? rotary_dim : 1);
  const bool aligned = (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0;
  if (dtype == asb::kBFloat16 && aligned && dim % 8 == 0 && vdim % 8 == 0 && hd % 8 == 0 && row % 8 == 0 && rotary_dim % 16 == 0) {
    const int vectors = (H * maps + KV) * (hd / 8);
    asb::launch(qk_prepare_store_vec_kernel, T_, vectors >= 256 ? 256 : (vectors >= 128 ? 128 : 64), smem, stream, p);
    return asb::check_launch("qk_prepare_store");
  }
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(qk_prepare_store_kernel<T>, T_, 256, smem, stream, p));
  return asb::check_launch("qk_prepare_store");
}

extern "C" int asb_differential_combine(void* out, const void* a, int rows, int hd, int vdim, float lambda,
                                        float post, float eps, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (vdim < 1 || vdim > hd) return asb::fail("differential_combine: values of %d in heads of %d", vdim, hd);
  ASB_DISPATCH_DTYPE(dtype, T, asb::launch(differential_combine_kernel<T>, (rows + 7) / 8, 256, 0, stream, (T*)out,
                                           (const T*)a, rows, hd, vdim, lambda, post, eps));
  return asb::check_launch("differential_combine");
}
