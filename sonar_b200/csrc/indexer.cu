// DeepSeek sparse-attention indexer: per query token, score every earlier key of its sequence with a
// light multi-head dot product and keep the positions of the best `k` keys.
//
//   logits[t, j] = Σ_h w[t, h] · relu( q[t, h, :] · key[j, :] )        j ≤ pos[t]   (64 heads, dim 128)
//   topk[t, :]   = positions of the k largest logits (any order), −1 padded when fewer exist
//
// Keys live in the paged latent cache: the indexer key of a token is `key_off` elements into its cache
// row.  The logits kernel is bandwidth-bound on those keys (256 B per key per query token): one CTA
// takes one query token and 256 keys, each warp runs mma.sync m16n8k16 on 16 keys × 64 heads × 128 dims
// from shared memory and reduces over heads in registers.  The selection kernel is a 4-pass 8-bit radix
// select over the row (L2-resident) followed by one gather pass.
//
// Behavioural parity: the reference computes these logits with DeepGEMM fp8 MQA-logits kernels
// (aphrodite/model_executor/layers/sparse_attn_indexer.py:576,707) and selects with topKPerRow
// (csrc/libtorch_stable/sampler.cu:545,569); this file is an independent bf16 formulation.
#include "common.cuh"

namespace sonar {
namespace {

constexpr int IH = 64;            // indexer heads
constexpr int ID = 128;           // indexer head dim
constexpr int PAD = ID + 8;       // smem row stride (elements): conflict-free fragment loads
constexpr int KEYS_PER_CTA = 256;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128) indexer_logits_kernel(
    const __nv_bfloat16* __restrict__ q, const float* __restrict__ w, const __nv_bfloat16* __restrict__ cache,
    long row_elems, int key_off, int block_size, const int* __restrict__ block_tables, long bt_stride,
    const int* __restrict__ token_seq, const long* __restrict__ positions, float* __restrict__ logits, long ld) {
  __shared__ __align__(16) __nv_bfloat16 q_s[IH * PAD];
  __shared__ __align__(16) __nv_bfloat16 k_s[4][16 * PAD];
  __shared__ float w_s[IH];
  const int t = blockIdx.y;
  const int j0 = blockIdx.x * KEYS_PER_CTA;
  const long pos = positions[t];
  float* out = logits + (long)t * ld + j0;
  if (j0 > pos) {   // nothing visible in this range
    for (int i = threadIdx.x; i < KEYS_PER_CTA; i += blockDim.x) out[i] = -INFINITY;
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // stage q[t] (64 × 128) and w[t]
  const uint4* qg = reinterpret_cast<const uint4*>(q + (long)t * IH * ID);
  for (int i = threadIdx.x; i < IH * (ID / 8); i += blockDim.x) {
    const int r = i / (ID / 8), c = i % (ID / 8);
    *reinterpret_cast<uint4*>(&q_s[r * PAD + c * 8]) = qg[i];
  }
  if (threadIdx.x < IH) w_s[threadIdx.x] = w[(long)t * IH + threadIdx.x];
  __syncthreads();
  const int* bt = block_tables + (long)token_seq[t] * bt_stride;
  const int gr = lane >> 2, gc = lane & 3;       // fragment row group / column pair
  __nv_bfloat16* ks = k_s[warp];
  for (int it = 0; it < KEYS_PER_CTA / 64; ++it) {
    const int kbase = j0 + it * 64 + warp * 16;  // this warp's 16 keys
    // load 16 keys × 256 B: 256 chunks of 16 B, 8 per lane
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int chunk = lane + i * 32;
      const int r = chunk >> 4, c = chunk & 15;
      const long j = (long)kbase + r;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (j <= pos) {
        const long blk = bt[j / block_size];
        const __nv_bfloat16* src = cache + (blk * block_size + (j % block_size)) * row_elems + key_off;
        v = *reinterpret_cast<const uint4*>(src + c * 8);
      }
      *reinterpret_cast<uint4*>(&ks[r * PAD + c * 8]) = v;
    }
    __syncwarp();
    float acc[IH / 8][4];
#pragma unroll
    for (int n = 0; n < IH / 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < ID / 16; ++kk) {
      uint32_t a[4];
      const int col = kk * 16 + gc * 2;
      a[0] = *reinterpret_cast<const uint32_t*>(&ks[gr * PAD + col]);
      a[1] = *reinterpret_cast<const uint32_t*>(&ks[(gr + 8) * PAD + col]);
      a[2] = *reinterpret_cast<const uint32_t*>(&ks[gr * PAD + col + 8]);
      a[3] = *reinterpret_cast<const uint32_t*>(&ks[(gr + 8) * PAD + col + 8]);
#pragma unroll
      for (int n = 0; n < IH / 8; ++n) {
        uint32_t b[2];
        const int head = n * 8 + gr;
        b[0] = *reinterpret_cast<const uint32_t*>(&q_s[head * PAD + col]);
        b[1] = *reinterpret_cast<const uint32_t*>(&q_s[head * PAD + col + 8]);
        mma_bf16_16816(acc[n], a, b);
      }
    }
    float s0 = 0.f, s1 = 0.f;      // keys gr and gr + 8
#pragma unroll
    for (int n = 0; n < IH / 8; ++n) {
      const float w0 = w_s[n * 8 + gc * 2], w1 = w_s[n * 8 + gc * 2 + 1];
      s0 += w0 * fmaxf(acc[n][0], 0.f) + w1 * fmaxf(acc[n][1], 0.f);
      s1 += w0 * fmaxf(acc[n][2], 0.f) + w1 * fmaxf(acc[n][3], 0.f);
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if (gc == 0) {
      const int o = it * 64 + warp * 16 + gr;
      out[o] = ((long)kbase + gr <= pos) ? s0 : -INFINITY;
      out[o + 8] = ((long)kbase + gr + 8 <= pos) ? s1 : -INFINITY;
    }
    __syncwarp();
  }
}

// order-preserving map float → uint32 (larger float ⇒ larger key)
__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA per row.  n = positions[t] + 1 valid entries; writes k indices (−1 padded).
__global__ void __launch_bounds__(512) indexer_topk_kernel(const float* __restrict__ logits, long ld,
                                                           const long* __restrict__ positions, int k,
                                                           int* __restrict__ out) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_need, s_gt, s_eq;
  const int t = blockIdx.x;
  const float* row = logits + (long)t * ld;
  int* o = out + (long)t * k;
  long n_l = positions[t] + 1;
  const int n = (int)(n_l < ld ? n_l : ld);
  if (n <= k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) o[i] = i < n ? i : -1;
    return;
  }
  if (threadIdx.x == 0) { s_prefix = 0u; s_mask = 0u; s_need = k; }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = fkey(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_need = need;                              // how many to take inside bin b
      s_prefix = prefix | ((uint32_t)b << shift);
      s_mask = mask | (255u << shift);
    }
    __syncthreads();
  }
  // s_prefix is now the key of the k-th largest value; s_need of the entries equal to it are taken
  const uint32_t thr = s_prefix;
  const int need_eq = s_need;
  if (threadIdx.x == 0) { s_gt = 0; s_eq = 0; }
  __syncthreads();
  const int n_gt = k - need_eq;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t key = fkey(row[i]);
    if (key > thr) {
      const int p = atomicAdd(&s_gt, 1);
      if (p < n_gt) o[p] = i;
    } else if (key == thr) {
      const int p = atomicAdd(&s_eq, 1);
      if (p < need_eq) o[n_gt + p] = i;
    }
  }
}

}  // namespace
}  // namespace sonar

using namespace sonar;

// q [T, 64, 128] bf16 contiguous, w [T, 64] fp32, cache rows of row_elems bf16 with the key at key_off,
// logits [T, ld] fp32 with ld a multiple of 256 covering the longest sequence.
SONAR_API int sonar_indexer_logits(const void* q, const float* w, const void* cache, long row_elems, int key_off,
                                   int block_size, const int* block_tables, long bt_stride, const int* token_seq,
                                   const long* positions, float* logits, long ld, int T, int heads, int dim,
                                   cudaStream_t s) {
  if (T == 0) return SONAR_OK;
  if (heads != IH || dim != ID || ld % KEYS_PER_CTA || key_off % 8 || row_elems % 8) return SONAR_BAD_ARG;
  if (T > 65535) return SONAR_TOO_LARGE;
  dim3 grid((unsigned)(ld / KEYS_PER_CTA), T);
  indexer_logits_kernel<<<grid, 128, 0, s>>>((const __nv_bfloat16*)q, w, (const __nv_bfloat16*)cache, row_elems,
                                             key_off, block_size, block_tables, bt_stride, token_seq, positions,
                                             logits, ld);
  return check_launch();
}

SONAR_API int sonar_indexer_topk(const float* logits, long ld, const long* positions, int k, int* out, int T,
                                 cudaStream_t s) {
  if (T == 0) return SONAR_OK;
  if (k <= 0) return SONAR_BAD_ARG;
  indexer_topk_kernel<<<T, 512, 0, s>>>(logits, ld, positions, k, out);
  return check_launch();
}
