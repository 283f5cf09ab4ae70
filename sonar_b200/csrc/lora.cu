// Batched-gather matrix-vector kernels for multi-adapter LoRA: every token row picks its own adapter.
//
//   shrink:  v[t, j]        = Σ_k A[slot[t], j, k] · x[t, k]          (rank r rows, K = layer input)
//   expand:  y[t, off + n] += Σ_j B[slot[t], n, j] · v[t, j]          (N = layer output slice, r small)
//
// slot[t] < 0 means "no adapter": the token is skipped.  Both kernels are bandwidth-bound on the
// adapter matrices (re-read per token, L2-resident), use 16-byte loads and fp32 accumulation; the
// LoRA scale α/r is folded into B when the adapter is loaded.
//
// Behavioural parity with the reference's Punica bgmv (csrc/punica/bgmv/bgmv_impl.cuh) and its
// shrink/expand Triton ops (aphrodite/lora/ops/triton_ops) — not code.
#include "common.cuh"

namespace sonar {
namespace {

// grid (T), block 256: warp w handles rank rows j = w, w+8, …
template <typename T>
__global__ void __launch_bounds__(256) lora_shrink_kernel(const T* __restrict__ x, long x_stride,
                                                          const T* __restrict__ A, long a_slot_stride,
                                                          const int* __restrict__ slots, float* __restrict__ v,
                                                          int r, int K) {
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint4* xv = reinterpret_cast<const uint4*>(x + (long)t * x_stride);
  const T* a0 = A + (long)slot * a_slot_stride;
  const int nvec = K >> 3;
  for (int j = warp; j < r; j += 8) {
    const uint4* av = reinterpret_cast<const uint4*>(a0 + (long)j * K);
    float acc = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      float a[8], b[8];
      unpack8<T>(av[i], a);
      unpack8<T>(xv[i], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += a[e] * b[e];
    }
    acc = warp_sum(acc);
    if (lane == 0) v[(long)t * r + j] = acc;
  }
}

// grid (T, ceil(N / 256)), block 256: thread n owns one output channel.
template <typename T>
__global__ void __launch_bounds__(256) lora_expand_kernel(const float* __restrict__ v, const T* __restrict__ B,
                                                          long b_slot_stride, const int* __restrict__ slots,
                                                          T* __restrict__ y, long y_stride, int y_off, int N, int r) {
  __shared__ float vs[256];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  if (threadIdx.x < r) vs[threadIdx.x] = v[(long)t * r + threadIdx.x];
  __syncthreads();
  const int n = blockIdx.y * 256 + threadIdx.x;
  if (n >= N) return;
  const uint4* bv = reinterpret_cast<const uint4*>(B + (long)slot * b_slot_stride + (long)n * r);
  float acc = 0.f;
  for (int i = 0; i < (r >> 3); ++i) {
    float b[8];
    unpack8<T>(bv[i], b);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += b[e] * vs[i * 8 + e];
  }
  T* dst = y + (long)t * y_stride + y_off + n;
  *dst = from_f<T>(to_f<T>(*dst) + acc);
}

}  // namespace
}  // namespace sonar

using namespace sonar;

// A: [slots, r, K]; v: [T, r] fp32 scratch
SONAR_API int sonar_lora_shrink(const void* x, long x_stride, const void* A, const int* slots, float* v, int T, int r,
                                int K, int dtype, cudaStream_t s) {
  if (T == 0) return SONAR_OK;
  if (K % 8 || x_stride % 8 || r <= 0 || r > 256) return SONAR_BAD_ARG;
  SONAR_DISPATCH_HALF(dtype, T_, {
    lora_shrink_kernel<T_><<<T, 256, 0, s>>>((const T_*)x, x_stride, (const T_*)A, (long)r * K, slots, v, r, K);
    return check_launch();
  });
}

// B: [slots, N, r]; y[t, y_off : y_off + N] += B[slot] · v[t]
SONAR_API int sonar_lora_expand(const float* v, const void* B, const int* slots, void* y, long y_stride, int y_off,
                                int T, int N, int r, int dtype, cudaStream_t s) {
  if (T == 0 || N == 0) return SONAR_OK;
  if (r % 8 || r <= 0 || r > 256) return SONAR_BAD_ARG;
  dim3 grid(T, (N + 255) / 256);
  SONAR_DISPATCH_HALF(dtype, T_, {
    lora_expand_kernel<T_><<<grid, 256, 0, s>>>(v, (const T_*)B, (long)N * r, slots, (T_*)y, y_stride, y_off, N, r);
    return check_launch();
  });
}
