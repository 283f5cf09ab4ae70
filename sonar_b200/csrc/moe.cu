// Mixture-of-experts routing and token permutation kernels.
//
//  topk_route      softmax or sigmoid scores over E experts, optional selection bias and expert groups
//                  (DeepSeek: keep the topk_group best groups by top-2 score sum), top-k ids + weights
//                  (optionally renormalised, scaled).  One warp per token.
//  moe_align       count tokens per (local) expert, pad each expert's segment to a multiple of 128 rows
//                  so GEMM tiles never straddle experts, and give every (token, slot) pair its row in the
//                  expert-sorted order; also writes the expert id of every 128-row block.
//  moe_gather      A_perm[row] = x[token of row] (rows of padding are zero-filled).
//  moe_combine     out[token] = Σ_slots weight · Y[row(token, slot)]; the destination of each token row may
//                  be a peer's partial-sum buffer (expert parallelism: the weighted combine and the
//                  return trip of the all-to-all are one kernel), followed by a completion flag.
//
// Behavioural parity: reference csrc/libtorch_stable/moe/topk_softmax_kernels.cu:645, grouped_topk_kernels.cu:525,
// moe_align_sum_kernels.cu:26-587, moe_permute_unpermute_op.cu.
#include "common.cuh"

namespace sonar {
namespace {

constexpr int MAX_E_PER_LANE = 16;   // experts ≤ 512
constexpr int MAX_K = 32;

struct RouteParams {
  const void* logits; int logits_dtype;   // [T, E]
  const float* bias;                      // [E] selection bias or null
  int T, E, k, n_group, topk_group, renorm, sigmoid;
  float scale;
  float* weights; int* ids;               // [T, k]
};

template <typename T>
__global__ void __launch_bounds__(256) topk_route_kernel(const RouteParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.T) return;
  const T* row = reinterpret_cast<const T*>(p.logits) + (long)warp * p.E;
  float score[MAX_E_PER_LANE], sel[MAX_E_PER_LANE];
  const int per = (p.E + 31) / 32;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    int e = lane + i * 32;
    score[i] = (i < per && e < p.E) ? to_f<T>(row[e]) : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  if (p.sigmoid) {
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i)
      score[i] = score[i] == -INFINITY ? -INFINITY : 1.f / (1.f + __expf(-score[i]));
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      score[i] = score[i] == -INFINITY ? 0.f : __expf(score[i] - mx);
      sum += score[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      int e = lane + i * 32;
      score[i] = (i < per && e < p.E) ? score[i] / sum : -INFINITY;
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    int e = lane + i * 32;
    sel[i] = (i < per && e < p.E) ? score[i] + (p.bias ? p.bias[e] : 0.f) : -INFINITY;
  }
  if (p.n_group > 1) {
    // group score = sum of the group's two best selection scores (max when there is no bias); keep topk_group groups
    const int gsz = p.E / p.n_group;
    float gscore_mine = -INFINITY;             // lane g (< n_group) holds group g's score
    for (int g = 0; g < p.n_group; ++g) {
      float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i) {
        int e = lane + i * 32;
        if (i < per && e < p.E && e / gsz == g) {
          if (sel[i] > b1) { b2 = b1; b1 = sel[i]; } else if (sel[i] > b2) b2 = sel[i];
        }
      }
      // merge (b1, b2) pairs across lanes
      for (int o = 16; o > 0; o >>= 1) {
        float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        float n1 = fmaxf(b1, o1);
        float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      float gs = p.bias ? b1 + b2 : b1;
      if (lane == g) gscore_mine = gs;
    }
    unsigned keep = 0;
    for (int j = 0; j < p.topk_group; ++j) {
      float v = gscore_mine;
      int idx = lane;
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      keep |= 1u << idx;
      if (lane == idx) gscore_mine = -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      int e = lane + i * 32;
      if (i < per && e < p.E && !((keep >> (e / gsz)) & 1u)) sel[i] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < p.k; ++j) {
    float v = -INFINITY, sc = 0.f;
    int idx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      int e = lane + i * 32;
      if (i < per && e < p.E && (sel[i] > v || (sel[i] == v && e < idx))) { v = sel[i]; idx = e; sc = score[i]; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o), os = __shfl_xor_sync(0xffffffffu, sc, o);
      int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; sc = os; }
    }
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i)
      if (lane + i * 32 == idx) sel[i] = -INFINITY;
    wsum += sc;
    if (lane == j) { my_w = sc; my_id = idx; }
  }
  if (lane < p.k) {
    float w = p.renorm ? my_w / (wsum + 1e-20f) : my_w;
    p.weights[(long)warp * p.k + lane] = w * p.scale;
    p.ids[(long)warp * p.k + lane] = my_id;
  }
}

// ---- alignment ---------------------------------------------------------------------------------
// counts[e]: pairs routed to local expert e.  ids are global expert ids; expert_map (or null) maps them to
// local ids (-1: not held here).
__global__ void moe_count_kernel(const int* ids, const int* expert_map, int n_pairs, int* counts) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  int e = ids[i];
  if (expert_map) e = expert_map[e];
  if (e >= 0) atomicAdd(counts + e, 1);
}
// One block: padded exclusive scan → offsets[e], cursor[e] = offsets[e]; block_expert for every 128-row block;
// meta[0] = number of 128-row blocks, meta[1] = padded rows.  Also resets counts for the next call.
__global__ void moe_scan_kernel(int* counts, int n_experts, int* offsets, int* cursor, int* block_expert, int* meta,
                                int max_blocks) {
  __shared__ int s_off[513];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < n_experts; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[n_experts] = acc;
    meta[0] = min(acc / 128, max_blocks);
    meta[1] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    offsets[e] = s_off[e];
    cursor[e] = s_off[e];
    for (int b = s_off[e] / 128; b < s_off[e + 1] / 128 && b < max_blocks; ++b) block_expert[b] = e;
    counts[e] = 0;
  }
}
// row_of[pair] = row in the expert-sorted order (-1 if the expert is not local); token_of[row] = token (-1 padding)
__global__ void moe_scatter_kernel(const int* ids, const int* expert_map, int n_pairs, int k, int* cursor,
                                   int* row_of, int* token_of) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  int e = ids[i];
  if (expert_map) e = expert_map[e];
  int row = -1;
  if (e >= 0) {
    row = atomicAdd(cursor + e, 1);
    token_of[row] = i / k;
  }
  row_of[i] = row;
}
__global__ void fill_kernel(int* p, int n, int v) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

template <typename T>
__global__ void __launch_bounds__(256) moe_gather_kernel(const T* __restrict__ x, long x_stride, const int* token_of,
                                                         const int* meta, T* __restrict__ out, int H) {
  const int row = blockIdx.x;
  if (row >= meta[1]) return;
  const int tok = token_of[row];
  uint4* dst = reinterpret_cast<uint4*>(out + (long)row * H);
  const uint4* src = reinterpret_cast<const uint4*>(x + (long)(tok < 0 ? 0 : tok) * x_stride);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) dst[v] = tok < 0 ? make_uint4(0, 0, 0, 0) : src[v];
}

struct CombineParams {
  const void* y;            // [rows, H] expert outputs in sorted order
  const int* row_of;        // [T, k]
  const float* weights;     // [T, k]
  int T, k, H;
  void* out;                // local destination [T, H] (dst_ptrs == null)
  void* const* dst_ptrs;    // [tp] peer partial-slot bases: token t goes to dst_ptrs[t / shard_rows] row t % shard_rows
  int shard_rows;
  int* local_done;          // [tp] arrival counters
  int* const* flag_ptrs;    // [tp] remote flags
  int seq; const int* seq_base;
};

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineParams p) {
  const int t = blockIdx.x;
  const T* y = reinterpret_cast<const T*>(p.y);
  T* dst;
  int d = 0;
  if (p.dst_ptrs) {
    d = t / p.shard_rows;
    dst = reinterpret_cast<T*>(p.dst_ptrs[d]) + (long)(t - d * p.shard_rows) * p.H;
  } else {
    dst = reinterpret_cast<T*>(p.out) + (long)t * p.H;
  }
  __shared__ int rows[MAX_K];
  __shared__ float ws[MAX_K];
  if (threadIdx.x < p.k) {
    rows[threadIdx.x] = p.row_of[(long)t * p.k + threadIdx.x];
    ws[threadIdx.x] = p.weights[(long)t * p.k + threadIdx.x];
  }
  __syncthreads();
  for (int v = threadIdx.x; v < p.H / 8; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < p.k; ++j) {
      if (rows[j] < 0) continue;
      float f[8];
      unpack8<T>(reinterpret_cast<const uint4*>(y + (long)rows[j] * p.H)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += ws[j] * f[i];
    }
    reinterpret_cast<uint4*>(dst)[v] = pack8<T>(acc);
  }
  if (p.dst_ptrs) {
    __syncthreads();
    if (threadIdx.x == 0) {
    // ordering: the block barrier orders every thread's stores before this thread's release-atomic
    // (gpu scope: it completes only after the block's outstanding stores, remote ones included, are
    // acknowledged); the arrival that completes the count publishes with a system-scope release store,
    // which is cumulative over everything it learned of through the counter.  A system-scope fence per
    // block measured ≈ 6 µs on this machine and is not needed for that chain.
      const int expected = min(p.T, (d + 1) * p.shard_rows) - d * p.shard_rows;
      int prev;
      asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(p.local_done + d) : "memory");
      if (prev + 1 == expected) {
        p.local_done[d] = 0;
        const int seq = p.seq + (p.seq_base ? *p.seq_base : 0);
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flag_ptrs[d]), "r"(seq) : "memory");
      }
    }
  }
}

}  // namespace
}  // namespace sonar

using namespace sonar;

SONAR_API int sonar_topk_route(const void* logits, int logits_dtype, const float* bias, int T, int E, int k,
                               int n_group, int topk_group, int renorm, int sigmoid, float scale, float* weights,
                               int* ids, cudaStream_t s) {
  if (T == 0) return SONAR_OK;
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E || n_group > 32 || (n_group > 1 && E % n_group)) return SONAR_BAD_ARG;
  RouteParams p{logits, logits_dtype, bias, T, E, k, n_group, topk_group, renorm, sigmoid, scale, weights, ids};
  int blocks = (T + 7) / 8;
  if (logits_dtype == SONAR_F32) topk_route_kernel<float><<<blocks, 256, 0, s>>>(p);
  else if (logits_dtype == SONAR_BF16) topk_route_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p);
  else if (logits_dtype == SONAR_F16) topk_route_kernel<__half><<<blocks, 256, 0, s>>>(p);
  else return SONAR_BAD_ARG;
  return check_launch();
}

// counts (zero on entry, zero on exit), offsets, cursor: [n_experts]; block_expert: [max_blocks]; meta: [2];
// row_of: [T*k]; token_of: [max_blocks*128].
SONAR_API int sonar_moe_align(const int* ids, const int* expert_map, int T, int k, int n_experts, int* counts,
                              int* offsets, int* cursor, int* block_expert, int* meta, int* row_of, int* token_of,
                              int max_blocks, cudaStream_t s) {
  if (n_experts > 512) return SONAR_TOO_LARGE;
  const int n = T * k;
  fill_kernel<<<(max_blocks * 128 + 255) / 256, 256, 0, s>>>(token_of, max_blocks * 128, -1);
  if (n > 0) moe_count_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, expert_map, n, counts);
  moe_scan_kernel<<<1, 256, 0, s>>>(counts, n_experts, offsets, cursor, block_expert, meta, max_blocks);
  if (n > 0) moe_scatter_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, expert_map, n, k, cursor, row_of, token_of);
  return check_launch();
}

SONAR_API int sonar_moe_gather(const void* x, long x_stride, const int* token_of, const int* meta, void* out, int H,
                               int max_rows, int dtype, cudaStream_t s) {
  if (H % 8) return SONAR_BAD_ARG;
  if (max_rows == 0) return SONAR_OK;
  SONAR_DISPATCH_HALF(dtype, T, {
    moe_gather_kernel<T><<<max_rows, 256, 0, s>>>((const T*)x, x_stride, token_of, meta, (T*)out, H);
    return check_launch();
  });
}

SONAR_API int sonar_moe_combine(const void* y, const int* row_of, const float* weights, int T, int k, int H, void* out,
                                void* const* dst_ptrs, int shard_rows, int* local_done, int* const* flag_ptrs, int seq,
                                const int* seq_base, int dtype, cudaStream_t s) {
  if (H % 8 || k > MAX_K) return SONAR_BAD_ARG;
  if (T == 0) return SONAR_OK;
  CombineParams p{y, row_of, weights, T, k, H, out, dst_ptrs, shard_rows, local_done, flag_ptrs, seq, seq_base};
  SONAR_DISPATCH_HALF(dtype, T_, {
    moe_combine_kernel<T_><<<T, 256, 0, s>>>(p);
    return check_launch();
  });
}
