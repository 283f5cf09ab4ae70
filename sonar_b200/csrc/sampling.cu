// Sampling kernels: arg-max, and temperature + top-k / top-p / min-p + exponential-race draw in one
// kernel without sorting.
//
// One 1024-thread block per row of fp32 logits [B, V].  Truncation thresholds are found by radix
// selection over the order-preserving integer image of the scaled logits (8-bit digits, per-warp
// shared-memory histograms): counts give the k-th largest value (top-k); probability mass (Σ exp(l-max))
// gives the nucleus boundary (top-p, evaluated among top-k survivors, a token stays while the mass
// strictly above it is below top_p·Z); min-p is a fixed offset below the maximum.  The draw is
// argmax(l_i/T − log e_i), e_i ~ Exp(1) from a counter-based hash RNG keyed by (seed, row, step, i), or
// from a caller-supplied noise tensor (used by the numerics tests).  Rows with temperature 0 take the
// arg-max of the raw logits.  Rows without truncation run two passes (max, draw).
//
// Behavioural parity: reference v1/sample/ops/topk_topp_sampler.py:72-537 (which defers to FlashInfer or
// Triton kernels; it has no in-tree CUDA sampler).
#include "common.cuh"

namespace sonar {
namespace {

constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;

__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// uniform in (0,1) from (seed, row-seed, step, index)
__device__ __forceinline__ float uniform01(uint64_t seed, uint32_t step, uint32_t idx) {
  uint32_t h = mix32((uint32_t)seed ^ mix32((uint32_t)(seed >> 32) + 0x9e3779b9u));
  h = mix32(h ^ mix32(step + 0x85ebca6bu));
  h = mix32(h ^ mix32(idx + 0xc2b2ae35u));
  return ((h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = a;
  __syncthreads();
  if (w == 0) {
    ArgMax t = lane < WARPS ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = better(t, b);
    }
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  ArgMax r = red[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, long stride, int V,
                                                          long* __restrict__ out) {
  __shared__ ArgMax red[WARPS];
  const float* row = logits + blockIdx.x * stride;
  ArgMax a{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += THREADS) a = better(a, ArgMax{row[i], i});
  a = block_argmax(a, red);
  if (threadIdx.x == 0) out[blockIdx.x] = a.i;
}

// Radix selection.  MASS = false: key of the k-th largest element (target = k).
// MASS = true: smallest key x such that mass strictly above x is < target (among keys >= floor_key).
// Returns the selected key; *total (MASS only) receives the total mass among keys >= floor_key.
template <bool MASS>
__device__ uint32_t radix_select(const float* row, int V, float inv_t, float maxv, float target, uint32_t floor_key,
                                 float* hist /* [WARPS][256] */, float* scratch /* [260] */, float* total) {
  uint32_t prefix = 0, prefix_mask = 0;
  float above = 0.f;  // count / mass strictly above the current prefix bucket
  const int w = threadIdx.x >> 5;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < WARPS * 256; i += THREADS) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += THREADS) {
      float l = row[i] * inv_t;
      uint32_t k = fkey(l);
      if ((k & prefix_mask) == prefix && k >= floor_key) {
        float add = MASS ? __expf(l - maxv) : 1.f;
        atomicAdd(&hist[w * 256 + ((k >> shift) & 255u)], add);
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      float s = 0.f;
      for (int ww = 0; ww < WARPS; ++ww) s += hist[ww * 256 + threadIdx.x];
      scratch[threadIdx.x] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float cum = above;
      int sel = 0;
      float tgt = target;
      if (MASS && shift == 24) {
        float z = 0.f;
        for (int b = 0; b < 256; ++b) z += scratch[b];
        *total = z;
        scratch[258] = z;
      }
      if (MASS) tgt = target * scratch[258];
      for (int b = 255; b >= 0; --b) {
        float c = scratch[b];
        if (c > 0.f && cum + c >= tgt) { sel = b; break; }
        cum += c;
        if (b == 0) sel = 0;
      }
      scratch[256] = __uint_as_float((uint32_t)sel);
      scratch[257] = cum;
    }
    __syncthreads();
    uint32_t sel = __float_as_uint(scratch[256]);
    above = scratch[257];
    prefix |= sel << shift;
    prefix_mask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(
    const float* __restrict__ logits, long stride, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ noise, long noise_stride, const long* __restrict__ seeds, uint32_t step,
    long* __restrict__ out) {
  __shared__ ArgMax red[WARPS];
  __shared__ float scratch[260];
  extern __shared__ float hist[];
  const int r = blockIdx.x;
  const float* row = logits + r * stride;
  const float T = temperature[r];
  if (T < 1e-5f) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += THREADS) a = better(a, ArgMax{row[i], i});
    a = block_argmax(a, red);
    if (threadIdx.x == 0) out[r] = a.i;
    return;
  }
  const float inv_t = 1.f / T;
  const int k = top_k ? top_k[r] : 0;
  const float p = top_p ? top_p[r] : 1.f;
  const float mp = min_p ? min_p[r] : 0.f;
  uint32_t floor_key = 0;
  if ((k > 0 && k < V) || p < 1.f || mp > 0.f) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += THREADS) a = better(a, ArgMax{row[i] * inv_t, i});
    a = block_argmax(a, red);
    const float maxv = a.v;
    if (k > 0 && k < V) floor_key = radix_select<false>(row, V, inv_t, maxv, (float)k, 0u, hist, scratch, nullptr);
    if (p < 1.f) {
      float z;
      uint32_t pk = radix_select<true>(row, V, inv_t, maxv, p, floor_key, hist, scratch, &z);
      floor_key = max(floor_key, pk);
    }
    if (mp > 0.f) floor_key = max(floor_key, fkey(maxv + __logf(mp)));
  }
  const uint64_t seed = seeds ? (uint64_t)seeds[r] : 0x243f6a8885a308d3ull + (uint64_t)r;
  const float* nz = noise ? noise + r * noise_stride : nullptr;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += THREADS) {
    float l = row[i] * inv_t;
    if (fkey(l) < floor_key) continue;
    float e = nz ? nz[i] : -__logf(uniform01(seed, step, (uint32_t)i));
    best = better(best, ArgMax{l - __logf(e), i});
  }
  best = block_argmax(best, red);
  if (threadIdx.x == 0) out[r] = best.i;
}

}  // namespace
}  // namespace sonar

using namespace sonar;

SONAR_API int sonar_argmax(const float* logits, long stride, int rows, int V, long* out, cudaStream_t s) {
  if (rows == 0) return SONAR_OK;
  argmax_kernel<<<rows, THREADS, 0, s>>>(logits, stride, V, out);
  return check_launch();
}

// seeds: per-row int64 RNG keys (null → fixed per-row constants); step: decorrelates successive calls.
SONAR_API int sonar_sample(const float* logits, long stride, int rows, int V, const float* temperature,
                           const int* top_k, const float* top_p, const float* min_p, const float* noise,
                           long noise_stride, const long* seeds, unsigned step, long* out, cudaStream_t s) {
  if (rows == 0) return SONAR_OK;
  const int smem = WARPS * 256 * sizeof(float);
  sample_kernel<<<rows, THREADS, smem, s>>>(logits, stride, V, temperature, top_k, top_p, min_p, noise, noise_stride,
                                            seeds, step, out);
  return check_launch();
}
