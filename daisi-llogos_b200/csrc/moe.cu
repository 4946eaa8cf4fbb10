// Mixture of experts: routing, the layout of a step's (token, choice) pairs by expert, the experts' two grouped products
// on the CUDA cores, and the weighted sum (argument blocks and the layout in kernel_args.h).
//
//   moe_route   : z = W_r x + b in float32 (x may be bfloat16), the `top` largest per token (ties: the lower index), weights
//                 softmax over the chosen z alone; or, by a RouterRule, sigmoid scores chosen within the best groups of
//                 experts and divided by their sum.
//   moe_plan    : one block counts the pairs of every expert, lays the experts' runs out one after another, each filled
//                 up to whole tiles, and gives every pair its row.  Which row of its expert's run a pair gets depends on
//                 the order in which the threads arrive; no result depends on it (a row's values come from its own token
//                 alone, and a token's rows are added in the order of its choices).
//   grouped products: a block takes one tile of rows (one expert) and a run of outputs: bfloat16 with rows that start on
//                 16-byte boundaries on the tensor cores (mma.sync), everything else on the CUDA cores.
//   moe_combine : out[n] = sum_k weight[n][k] y[row of (n, k)] + the shared expert's partial sums.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_moe_tile_rows() { return LLG_MOE_TILE; }
LLG_API int llg_moe_max_experts() { return LLG_MOE_MAX_EXPERTS; }
LLG_API int llg_moe_max_top() { return LLG_MOE_MAX_TOP; }

namespace {

// One warp turns a token's logits z[0 .. n_exp) (shared memory, overwritten) into its `top` experts and their weights by
// `rule` (RouterRule in kernel_args.h).  Ties go to the lower index.  gsc: n_exp floats of scratch beside z (group
// scores and the marks of the groups that stay).
__device__ __forceinline__ void choose_and_weigh(float* z, float* gsc, float* chosen, int n_exp, int top, const RouterRule& rule,
                                                 int* __restrict__ choice, float* __restrict__ weight, int lane) {
  if (rule.score == 2) {
    // scores: the softmax over every expert's logit
    float m = -INFINITY;
    for (int e = lane; e < n_exp; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float total = 0.f;
    for (int e = lane; e < n_exp; e += 32) {
      const float ev = expf(z[e] - m);
      z[e] = ev;
      total += ev;
    }
    total = warp_sum(total);
    for (int e = lane; e < n_exp; e += 32) z[e] = z[e] / total;
    __syncwarp();
  }
  if (rule.score == 1) {
    for (int e = lane; e < n_exp; e += 32) z[e] = 1.0f / (1.0f + expf(-z[e]));
    __syncwarp();
    if (rule.groups > 0) {
      const int per = n_exp / rule.groups;
      // a group's score: the sum of its group_top largest scores (a lane per group, the largest taken one after another)
      for (int g = lane; g < rule.groups; g += 32) {
        const float* zg = z + g * per;
        float total = 0.f, prev = INFINITY;
        int prev_i = -1;
        for (int t = 0; t < rule.group_top && t < per; ++t) {
          float best = -INFINITY;
          int arg = -1;
          for (int i = 0; i < per; ++i) {
            const float v = zg[i];
            const bool after = v < prev || (v == prev && i > prev_i);     // not taken yet
            if (after && v > best) { best = v; arg = i; }
          }
          if (arg < 0) break;
          total += best;
          prev = best;
          prev_i = arg;
        }
        gsc[g] = total;
      }
      __syncwarp();
      // the keep_groups best groups stay: their mark is 2 (no sum of scores reaches it), the others' scores fall to -1
      for (int k = 0; k < rule.keep_groups; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int g = lane; g < rule.groups; g += 32) {
          const float v = gsc[g];
          if (v <= (float)per && v > best) { best = v; arg = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
          if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0 && arg != 0x7fffffff) gsc[arg] = 2.0f * (float)per + 1.0f;
        __syncwarp();
      }
      for (int e = lane; e < n_exp; e += 32)
        if (gsc[e / per] <= (float)per) z[e] = -1.0f;
      __syncwarp();
    }
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < n_exp; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; arg = e; }          // a lane meets its experts in rising order: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;                 // nothing but -inf or NaN left: still a valid index
    if (lane == 0) {
      choice[k] = arg;
      chosen[k] = best;
      z[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (rule.score != 0) {
    // the chosen scores divided by their sum
    const float sv = lane < top ? chosen[lane] : 0.f;
    const float total = warp_sum(sv);
    if (lane < top) weight[lane] = sv / (total + rule.sum_eps) * rule.scale;
    return;
  }
  // softmax over the chosen logits; the first chosen is the largest
  const float m = chosen[0];
  float ev = lane < top ? expf(chosen[lane] - m) : 0.f;
  const float total = warp_sum(ev);
  if (lane < top) weight[lane] = ev / total;
}

// A token's logits z = W_r x + b with float32 sums, then choose_and_weigh.  With `extra` the matrix has one more row
// behind the experts': extra[n] = sigmoid(that row . x).
template <typename XT>
__global__ void __launch_bounds__(128) moe_route_kernel(const XT* __restrict__ x, const float* __restrict__ w,
                                                        const float* __restrict__ bias, int* __restrict__ choice,
                                                        float* __restrict__ weight, int hidden, int n_exp, int top,
                                                        RouterRule rule, float* __restrict__ extra) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* xs = sm;                   // [hidden]
  float* z = sm + hidden;           // [n_exp + 1], then [n_exp] of scratch
  __shared__ float chosen[LLG_MOE_MAX_TOP];
  const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = to_f32(x[(long long)n * hidden + i]);
  __syncthreads();
  const int rows = n_exp + (extra ? 1 : 0);
  for (int e = warp; e < rows; e += 4) {
    const float* we = w + (long long)e * hidden;
    float s = 0.f;
    for (int i = lane; i < hidden; i += 32) s = fmaf(we[i], xs[i], s);
    s = warp_sum(s);
    if (lane == 0) z[e] = s + (bias && e < n_exp ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  if (extra && lane == 0) extra[n] = 1.0f / (1.0f + expf(-z[n_exp]));
  choose_and_weigh(z, z + n_exp + 1, chosen, n_exp, top, rule, choice + (long long)n * top, weight + (long long)n * top, lane);
}

// The same choice from logits that a product has left as float32 partial sums [n_partials][n_tokens][width] (the router's
// matrix product on the tensor cores, where the checkpoint stores the router in the compute type; width = n_exp, or with
// `extra` n_exp + 1): a warp per token adds the partials and the bias, then chooses and weighs as moe_route does.
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, int n_partials, long long partial_stride,
                                                       const float* __restrict__ bias, int* __restrict__ choice,
                                                       float* __restrict__ weight, int n_tokens, int n_exp, int top,
                                                       RouterRule rule, float* __restrict__ extra) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  __shared__ float chosen_all[4][LLG_MOE_MAX_TOP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  if (n >= n_tokens) return;
  const int width = n_exp + (extra ? 1 : 0);
  float* z = sm + warp * (2 * n_exp + 1);
  for (int e = lane; e < width; e += 32) {
    float v = bias && e < n_exp ? bias[e] : 0.f;
    for (int s = 0; s < n_partials; ++s) v += logits[s * partial_stride + (long long)n * width + e];
    z[e] = v;
  }
  __syncwarp();
  if (extra && lane == 0) extra[n] = 1.0f / (1.0f + expf(-z[n_exp]));
  choose_and_weigh(z, z + n_exp + 1, chosen_all[warp], n_exp, top, rule, choice + (long long)n * top, weight + (long long)n * top,
                   lane);
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ choice, int n_pairs, int top, int n_exp,
                                                        int* __restrict__ row_of_pair, int* __restrict__ token_of_row,
                                                        int* __restrict__ tile_expert, int cap, int tile_rows) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int counts[LLG_MOE_MAX_EXPERTS], starts[LLG_MOE_MAX_EXPERTS], cursor[LLG_MOE_MAX_EXPERTS];
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int e = tid; e < n_exp; e += nt) counts[e] = cursor[e] = 0;
  for (int r = tid; r < cap; r += nt) token_of_row[r] = -1;
  for (int t = tid; t < cap / tile_rows; t += nt) tile_expert[t] = -1;
  __syncthreads();
  for (int p = tid; p < n_pairs; p += nt) {
    const int e = choice[p];
    if (e >= 0 && e < n_exp) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < n_exp; ++e) {
      starts[e] = at;
      at += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
    }
  }
  __syncthreads();
  for (int e = tid; e < n_exp; e += nt) {
    const int t0 = starts[e] / tile_rows, t1 = t0 + (counts[e] + tile_rows - 1) / tile_rows;
    for (int t = t0; t < t1; ++t) tile_expert[t] = e;
  }
  for (int p = tid; p < n_pairs; p += nt) {
    const int e = choice[p];
    int row = 0;
    if (e >= 0 && e < n_exp) {
      row = starts[e] + atomicAdd(&cursor[e], 1);
      token_of_row[row] = p / top;
    }
    row_of_pair[p] = row;
  }
}

constexpr int GT_O = 32, GT_K = 32;

template <typename XT, typename WT, typename YT, bool GATED>
__global__ void __launch_bounds__(256) grouped_linear_kernel(GroupedLinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[LLG_MOE_TILE][GT_K + 1];
  __shared__ float ws[GT_O][GT_K + 1];
  __shared__ float ws2[GATED ? GT_O : 1][GT_K + 1];
  __shared__ int src[LLG_MOE_TILE];
  const int tile = blockIdx.x;
  const int e = a.tile_expert[tile];
  if (e < 0) return;
  const int r0 = tile * LLG_MOE_TILE, o0 = blockIdx.y * GT_O;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  if (threadIdx.x < LLG_MOE_TILE) src[threadIdx.x] = a.token_of_row ? a.token_of_row[r0 + threadIdx.x] : r0 + threadIdx.x;
  const XT* x = (const XT*)a.x;
  const long long w_gs = a.w_group_stride ? a.w_group_stride : (long long)a.n_out * a.n_in;
  const WT* w = (const WT*)a.w + e * w_gs;
  const WT* w2 = GATED ? (const WT*)a.w2 + e * w_gs : nullptr;
  constexpr int RPT = LLG_MOE_TILE / 8;             // rows per thread
  float acc[RPT], acc2[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) acc[i] = acc2[i] = 0.f;
  for (int k0 = 0; k0 < a.n_in; k0 += GT_K) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < LLG_MOE_TILE * GT_K; idx += 256) {
      const int r = idx / GT_K, c = idx % GT_K;
      const int s = src[r], k = k0 + c;
      xs[r][c] = (s >= 0 && k < a.n_in) ? to_f32(x[(long long)s * a.n_in + k]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < GT_O * GT_K; idx += 256) {
      const int r = idx / GT_K, c = idx % GT_K;
      const int o = o0 + r, k = k0 + c;
      const bool in = o < a.n_out && k < a.n_in;
      ws[r][c] = in ? to_f32(w[(long long)o * a.n_in + k]) : 0.f;
      if (GATED) ws2[r][c] = in ? to_f32(w2[(long long)o * a.n_in + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GT_K; ++k) {
      const float wv = ws[tx][k];
      const float wv2 = GATED ? ws2[tx][k] : 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const float xv = xs[ty + 8 * i][k];
        acc[i] = fmaf(xv, wv, acc[i]);
        if (GATED) acc2[i] = fmaf(xv, wv2, acc2[i]);
      }
    }
  }
  const int o = o0 + tx;
  if (o >= a.n_out) return;
  YT* y = (YT*)a.y;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = r0 + ty + 8 * i;
    float v = acc[i];
    if (GATED) v = v / (1.0f + expf(-v)) * acc2[i];
    y[(long long)r * a.n_out + o] = from_f32<YT>(v);         // filling rows hold zeros
  }
}

// ---- the grouped products on the tensor cores (bfloat16) ------------------------------------------------------------
//
// A block of four warps takes one tile of LLG_MOE_TILE rows (one expert) and MM_O outputs; the activations' rows (gathered
// through token_of_row) and the expert's matrix rows arrive in shared memory by 16-byte asynchronous copies, two stages
// deep, in k-blocks of MM_K; every warp owns MM_O / 4 outputs of all rows and multiplies with mma.sync m16n8k16 (bfloat16
// in, float32 sums).  GATED: a second matrix's tile beside the first, and silu(first) * second is what is stored.
constexpr int MM_O = 128, MM_K = 64, MM_PAD = 8;            // MM_PAD halves between rows: fragment loads meet no bank twice
constexpr int MM_LD = MM_K + MM_PAD;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 16 : 0;                          // 0: the 16 bytes are filled with zeros, src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename YT, bool GATED>
__global__ void __launch_bounds__(128) grouped_linear_mma_kernel(GroupedLinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char mm_smem[];
  typedef __nv_bfloat16 bf16;
  constexpr int A_HALVES = LLG_MOE_TILE * MM_LD, B_HALVES = MM_O * MM_LD;
  constexpr int STAGE_HALVES = A_HALVES + (GATED ? 2 : 1) * B_HALVES;
  bf16* base = reinterpret_cast<bf16*>(mm_smem);
  __shared__ int src[LLG_MOE_TILE];
  const int tile = blockIdx.x;
  const int e = a.tile_expert ? a.tile_expert[tile] : (int)blockIdx.z;
  if (e < 0) return;
  const int r0 = tile * LLG_MOE_TILE, o0 = blockIdx.y * MM_O;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (tid < LLG_MOE_TILE)
    src[tid] = a.token_of_row ? a.token_of_row[r0 + tid] : (a.n_rows == 0 || r0 + tid < a.n_rows) ? r0 + tid : -1;
  __syncthreads();
  const long long x_ld = a.x_row_stride ? a.x_row_stride : a.n_in, y_ld = a.y_row_stride ? a.y_row_stride : a.n_out;
  const bf16* x = (const bf16*)a.x + (long long)e * a.x_group_stride;
  const long long w_gs = a.w_group_stride ? a.w_group_stride : (long long)a.n_out * a.n_in;
  const bf16* w = (const bf16*)a.w + e * w_gs;
  const bf16* w2 = GATED ? (const bf16*)a.w2 + e * w_gs : nullptr;
  constexpr int CH = MM_K / 8;                                // 16-byte chunks in a row of a k-block
  auto load_stage = [&](int s, int k0) {
    bf16* As = base + s * STAGE_HALVES;
    bf16* Bs = As + A_HALVES;
    for (int idx = tid; idx < LLG_MOE_TILE * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH, k = k0 + c * 8;
      const int sr = src[r];
      const bool ok = sr >= 0 && k < a.n_in;
      cp_async16(As + r * MM_LD + c * 8, ok ? x + (long long)sr * x_ld + k : x, ok);
    }
    for (int idx = tid; idx < MM_O * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH, k = k0 + c * 8, o = o0 + r;
      const bool ok = o < a.n_out && k < a.n_in;
      const long long off = ok ? (long long)o * a.n_in + k : 0;
      cp_async16(Bs + r * MM_LD + c * 8, w + off, ok);
      if (GATED) cp_async16(Bs + B_HALVES + r * MM_LD + c * 8, w2 + off, ok);
    }
  };
  constexpr int MT = LLG_MOE_TILE / 16, NT = MM_O / 4 / 8;    // 16-row tiles of the block, 8-output tiles of a warp
  float acc[MT][NT][4], acc2[GATED ? MT : 1][GATED ? NT : 1][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[i][j][c] = 0.f;
        if (GATED) acc2[i][j][c] = 0.f;
      }
  const int nkb = (a.n_in + MM_K - 1) / MM_K;
  load_stage(0, 0);
  cp_async_commit();
  for (int kb = 0; kb < nkb; ++kb) {
    if (kb + 1 < nkb) {
      load_stage((kb + 1) & 1, (kb + 1) * MM_K);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* As = base + (kb & 1) * STAGE_HALVES;
    const bf16* Bs = As + A_HALVES + warp * (MM_O / 4) * MM_LD;
#pragma unroll
    for (int ks = 0; ks < MM_K; ks += 16) {
      unsigned af[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const bf16* ap = As + (i * 16 + g) * MM_LD + ks + 2 * t;
        af[i][0] = *reinterpret_cast<const unsigned*>(ap);
        af[i][1] = *reinterpret_cast<const unsigned*>(ap + 8 * MM_LD);
        af[i][2] = *reinterpret_cast<const unsigned*>(ap + 8);
        af[i][3] = *reinterpret_cast<const unsigned*>(ap + 8 * MM_LD + 8);
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const bf16* bp = Bs + (j * 8 + g) * MM_LD + ks + 2 * t;
        const unsigned b0 = *reinterpret_cast<const unsigned*>(bp), b1 = *reinterpret_cast<const unsigned*>(bp + 8);
#pragma unroll
        for (int i = 0; i < MT; ++i) mma_bf16(acc[i][j], af[i], b0, b1);
        if (GATED) {
          const unsigned c0 = *reinterpret_cast<const unsigned*>(bp + B_HALVES), c1 = *reinterpret_cast<const unsigned*>(bp + B_HALVES + 8);
#pragma unroll
          for (int i = 0; i < MT; ++i) mma_bf16(acc2[i][j], af[i], c0, c1);
        }
      }
    }
    __syncthreads();                                          // the stage is free for the copies of the step after next
  }
  YT* y = (YT*)a.y + (long long)e * a.y_group_stride;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = r0 + i * 16 + g + (c >> 1) * 8;
        const int o = o0 + warp * (MM_O / 4) + j * 8 + 2 * t + (c & 1);
        if (o >= a.n_out || (a.n_rows && r >= a.n_rows)) continue;
        float v = acc[i][j][c];
        if (GATED) v = v / (1.0f + expf(-v)) * acc2[i][j][c];
        y[(long long)r * y_ld + o] = from_f32<YT>(v);
      }
}

// out[r] = x[token_of_row[r]] (zeros for a filling row): the rows of the layout as one matrix, for a product that reads its
// first operand by tensor copies.  16 bytes a thread.
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of_row, uint4* __restrict__ out,
                                       int rows, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * chunks) return;
  const int r = (int)(i / chunks), c = (int)(i % chunks);
  const int t = token_of_row[r];
  out[i] = t >= 0 ? x[(long long)t * chunks + c] : make_uint4(0u, 0u, 0u, 0u);
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ weight, const float* __restrict__ shared, int n_shared,
                                   long long shared_stride, const float* __restrict__ shared_scale, float* __restrict__ out,
                                   int hidden, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < hidden; d += gridDim.y * blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = row_of_pair[(long long)n * top + k];
      v = fmaf(weight[(long long)n * top + k], y[(long long)row * hidden + d], v);
    }
    float sh = 0.f;
    for (int s = 0; s < n_shared; ++s) sh += shared[s * shared_stride + (long long)n * hidden + d];
    out[(long long)n * hidden + d] = v + (shared_scale ? shared_scale[n] * sh : sh);
  }
}

// The same with four columns a thread (rows that start on 16-byte boundaries): every load of a thread is independent of
// the others, so the few rows of a decode step are not a chain of waits.
__global__ void moe_combine_vec4_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair,
                                        const float* __restrict__ weight, const float* __restrict__ shared, int n_shared,
                                        long long shared_stride, const float* __restrict__ shared_scale,
                                        float* __restrict__ out, int hidden, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (d >= hidden) return;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < top; ++k) {
    const int row = row_of_pair[(long long)n * top + k];
    const float wk = weight[(long long)n * top + k];
    const float4 u = *reinterpret_cast<const float4*>(y + (long long)row * hidden + d);
    v.x = fmaf(wk, u.x, v.x); v.y = fmaf(wk, u.y, v.y); v.z = fmaf(wk, u.z, v.z); v.w = fmaf(wk, u.w, v.w);
  }
  float4 sh = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < n_shared; ++s) {
    const float4 u = *reinterpret_cast<const float4*>(shared + s * shared_stride + (long long)n * hidden + d);
    sh.x += u.x; sh.y += u.y; sh.z += u.z; sh.w += u.w;
  }
  const float sc = shared_scale ? shared_scale[n] : 1.0f;
  v.x = fmaf(sc, sh.x, v.x); v.y = fmaf(sc, sh.y, v.y); v.z = fmaf(sc, sh.z, v.z); v.w = fmaf(sc, sh.w, v.w);
  *reinterpret_cast<float4*>(out + (long long)n * hidden + d) = v;
}

}  // namespace

static int check_rule(const char* what, const RouterRule& r, int n_exp, int top) {
  LLG_REQUIRE(r.score >= 0 && r.score <= 2, "%s: score kind %d is not known", what, r.score);
  LLG_REQUIRE(r.groups >= 0 && (r.groups == 0 || r.score == 1), "%s: groups of experts go with sigmoid scores", what);
  if (r.groups > 0) {
    LLG_REQUIRE(n_exp % r.groups == 0 && r.keep_groups > 0 && r.keep_groups <= r.groups && r.group_top > 0,
                "%s: %d experts in %d groups of which %d stay, judged by %d scores", what, n_exp, r.groups, r.keep_groups, r.group_top);
    LLG_REQUIRE(top <= r.keep_groups * (n_exp / r.groups), "%s: top %d exceeds the experts of %d groups", what, top, r.keep_groups);
  }
  return 0;
}

// rule: null = the `top` largest logits weighted by a softmax over them.  extra: null, or [n_tokens] for the sigmoid of one
// more row of w behind the experts' rows.
LLG_API int llg_moe_route(const void* x, int x_dtype, const float* w, const float* bias, int* choice, float* weight,
                          int n_tokens, int hidden, int n_exp, int top, const RouterRule* rule, float* extra, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && hidden > 0, "moe_route: bad sizes");
  LLG_REQUIRE(n_exp > 0 && n_exp <= LLG_MOE_MAX_EXPERTS, "moe_route: %d experts are outside [1, %d]", n_exp, LLG_MOE_MAX_EXPERTS);
  LLG_REQUIRE(top > 0 && top <= n_exp && top <= LLG_MOE_MAX_TOP, "moe_route: top %d of %d experts (at most %d)", top, n_exp,
              LLG_MOE_MAX_TOP);
  const RouterRule r = rule ? *rule : RouterRule{0, 0, 0, 0, 1.0f, 0.0f};
  if (check_rule("moe_route", r, n_exp, top)) return 1;
  if (n_tokens == 0) return 0;
  const size_t smem = (size_t)(hidden + 2 * n_exp + 1) * sizeof(float);
  LLG_REQUIRE(smem <= 200 * 1024, "moe_route: rows of %d elements do not fit shared memory", hidden);
  if (x_dtype == LLG_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    llg_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(128), smem, stream, (const float*)x, w, bias, choice, weight, hidden,
               n_exp, top, r, extra);
  } else if (x_dtype == LLG_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    llg_launch(moe_route_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), smem, stream, (const __nv_bfloat16*)x, w, bias, choice,
               weight, hidden, n_exp, top, r, extra);
  } else {
    return llg_fail("moe_route: unknown dtype %d", x_dtype);
  }
  return llg_check_launch("moe_route");
}

// logits: [n_partials][n_tokens][n_exp], or with `extra` one more column behind the experts'.
LLG_API int llg_moe_topk(const float* logits, int n_partials, long long partial_stride, const float* bias, int* choice,
                         float* weight, int n_tokens, int n_exp, int top, const RouterRule* rule, float* extra, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && n_partials >= 1, "moe_topk: bad sizes");
  LLG_REQUIRE(n_exp > 0 && n_exp <= LLG_MOE_MAX_EXPERTS, "moe_topk: %d experts are outside [1, %d]", n_exp, LLG_MOE_MAX_EXPERTS);
  LLG_REQUIRE(top > 0 && top <= n_exp && top <= LLG_MOE_MAX_TOP, "moe_topk: top %d of %d experts (at most %d)", top, n_exp,
              LLG_MOE_MAX_TOP);
  const RouterRule r = rule ? *rule : RouterRule{0, 0, 0, 0, 1.0f, 0.0f};
  if (check_rule("moe_topk", r, n_exp, top)) return 1;
  if (n_tokens == 0) return 0;
  llg_launch(moe_topk_kernel, dim3((n_tokens + 3) / 4), dim3(128), (size_t)4 * (2 * n_exp + 1) * sizeof(float), stream, logits,
             n_partials, partial_stride, bias, choice, weight, n_tokens, n_exp, top, r, extra);
  return llg_check_launch("moe_topk");
}

LLG_API int llg_moe_plan(const int* choice, int n_pairs, int top, int n_exp, int* row_of_pair, int* token_of_row,
                         int* tile_expert, int cap, int tile_rows, cudaStream_t stream) {
  LLG_REQUIRE(tile_rows > 0, "moe_plan: tiles of %d rows", tile_rows);
  LLG_REQUIRE(n_exp > 0 && n_exp <= LLG_MOE_MAX_EXPERTS, "moe_plan: %d experts are outside [1, %d]", n_exp, LLG_MOE_MAX_EXPERTS);
  LLG_REQUIRE(top > 0 && n_pairs >= 0 && n_pairs % top == 0, "moe_plan: %d pairs, top %d", n_pairs, top);
  const long long need = ((long long)n_pairs + (long long)n_exp * (tile_rows - 1) + tile_rows - 1) / tile_rows * tile_rows;
  LLG_REQUIRE(cap % tile_rows == 0 && cap >= need, "moe_plan: %d rows, %lld needed (whole tiles)", cap, need);
  if (n_pairs == 0) return 0;
  llg_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, choice, n_pairs, top, n_exp, row_of_pair, token_of_row, tile_expert, cap,
             tile_rows);
  return llg_check_launch("moe_plan");
}

LLG_API int llg_grouped_linear(const GroupedLinearArgs* args, int x_dtype, int y_dtype, cudaStream_t stream) {
  const GroupedLinearArgs& a = *args;
  LLG_REQUIRE(a.rows >= 0 && a.rows % LLG_MOE_TILE == 0 && a.n_in > 0 && a.n_out > 0, "grouped_linear: bad sizes");
  if (a.rows == 0) return 0;
  const bool gated = a.w2 != nullptr;
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
  if (x_dtype == LLG_BF16 && a.n_in % 8 == 0 && aligned(a.x) && aligned(a.w) && aligned(a.w2)) {
    // the tensor-core kernel: 16-byte copies need rows that start on 16-byte boundaries
    dim3 mgrid(a.rows / LLG_MOE_TILE, (a.n_out + MM_O - 1) / MM_O);
    LLG_REQUIRE(mgrid.y <= 65535, "grouped_linear: too many outputs");
    const size_t smem = 2 * (size_t)(LLG_MOE_TILE * MM_LD + (gated ? 2 : 1) * MM_O * MM_LD) * sizeof(__nv_bfloat16);
#define MMA_LAUNCH(YT, G)                                                                                         \
  do {                                                                                                            \
    cudaError_t err = cudaFuncSetAttribute(grouped_linear_mma_kernel<YT, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (err != cudaSuccess) return llg_fail("grouped_linear: shared memory %zu: %s", smem, cudaGetErrorString(err)); \
    llg_launch(grouped_linear_mma_kernel<YT, G>, mgrid, dim3(128), smem, stream, a);                              \
  } while (0)
    if (y_dtype == LLG_BF16) {
      if (gated) MMA_LAUNCH(__nv_bfloat16, true); else MMA_LAUNCH(__nv_bfloat16, false);
    } else if (y_dtype == LLG_F32) {
      if (gated) MMA_LAUNCH(float, true); else MMA_LAUNCH(float, false);
    } else {
      return llg_fail("grouped_linear: unsupported output dtype %d", y_dtype);
    }
#undef MMA_LAUNCH
    return llg_check_launch("grouped_linear");
  }
  dim3 grid(a.rows / LLG_MOE_TILE, (a.n_out + GT_O - 1) / GT_O);
  LLG_REQUIRE(grid.y <= 65535, "grouped_linear: too many outputs");
  if (x_dtype == LLG_F32 && y_dtype == LLG_F32) {
    if (gated) llg_launch(grouped_linear_kernel<float, float, float, true>, grid, dim3(256), 0, stream, a);
    else llg_launch(grouped_linear_kernel<float, float, float, false>, grid, dim3(256), 0, stream, a);
  } else if (x_dtype == LLG_BF16 && y_dtype == LLG_BF16) {
    if (gated) llg_launch(grouped_linear_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, true>, grid, dim3(256), 0, stream, a);
    else llg_launch(grouped_linear_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, false>, grid, dim3(256), 0, stream, a);
  } else if (x_dtype == LLG_BF16 && y_dtype == LLG_F32) {
    if (gated) llg_launch(grouped_linear_kernel<__nv_bfloat16, __nv_bfloat16, float, true>, grid, dim3(256), 0, stream, a);
    else llg_launch(grouped_linear_kernel<__nv_bfloat16, __nv_bfloat16, float, false>, grid, dim3(256), 0, stream, a);
  } else {
    return llg_fail("grouped_linear: unsupported dtypes x=%d y=%d", x_dtype, y_dtype);
  }
  return llg_check_launch("grouped_linear");
}

// y[n][h][:] = w[h] x[n][h][:] on the tensor cores (bfloat16; x rows on 16-byte boundaries): the grouped kernel with the
// head as the group.  The caller has checked the alignment (llg_head_linear_mma_supported).
LLG_API int llg_head_linear_mma_supported(const void* x, long long x_token_stride, long long x_head_stride, const void* w, int n_in) {
  return n_in % 8 == 0 && x_token_stride % 8 == 0 && x_head_stride % 8 == 0 && ((uintptr_t)x & 15u) == 0 && ((uintptr_t)w & 15u) == 0;
}

LLG_API int llg_head_linear_mma(const void* x, long long x_token_stride, long long x_head_stride, const void* w, void* y,
                                long long y_token_stride, long long y_head_stride, int n_tokens, int nh, int n_in, int n_out,
                                int y_dtype, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && nh > 0 && nh <= 65535 && n_in > 0 && n_out > 0, "head_linear: bad sizes");
  LLG_REQUIRE(llg_head_linear_mma_supported(x, x_token_stride, x_head_stride, w, n_in),
              "head_linear: the tensor-core kernel wants rows that start on 16-byte boundaries");
  if (n_tokens == 0) return 0;
  GroupedLinearArgs a;
  memset(&a, 0, sizeof(a));
  a.x = x;
  a.w = w;
  a.y = y;
  a.rows = (n_tokens + LLG_MOE_TILE - 1) / LLG_MOE_TILE * LLG_MOE_TILE;
  a.n_in = n_in;
  a.n_out = n_out;
  a.x_row_stride = x_token_stride;
  a.y_row_stride = y_token_stride;
  a.x_group_stride = x_head_stride;
  a.y_group_stride = y_head_stride;
  a.n_rows = n_tokens;
  dim3 grid(a.rows / LLG_MOE_TILE, (n_out + MM_O - 1) / MM_O, nh);
  LLG_REQUIRE(grid.y <= 65535, "head_linear: too many outputs");
  const size_t smem = 2 * (size_t)(LLG_MOE_TILE * MM_LD + MM_O * MM_LD) * sizeof(__nv_bfloat16);
#define HEAD_LAUNCH(YT)                                                                                                       \
  do {                                                                                                                        \
    cudaError_t err = cudaFuncSetAttribute(grouped_linear_mma_kernel<YT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (err != cudaSuccess) return llg_fail("head_linear: shared memory %zu: %s", smem, cudaGetErrorString(err));             \
    llg_launch(grouped_linear_mma_kernel<YT, false>, grid, dim3(128), smem, stream, a);                                       \
  } while (0)
  if (y_dtype == LLG_BF16) HEAD_LAUNCH(__nv_bfloat16);
  else if (y_dtype == LLG_F32) HEAD_LAUNCH(float);
  else return llg_fail("head_linear: unknown output type %d", y_dtype);
#undef HEAD_LAUNCH
  return llg_check_launch("head_linear");
}

LLG_API int llg_moe_gather_rows(const void* x, const int* token_of_row, void* out, int rows, int row_bytes, cudaStream_t stream) {
  LLG_REQUIRE(rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0 && ((uintptr_t)x & 15u) == 0 && ((uintptr_t)out & 15u) == 0,
              "moe_gather_rows: rows of %d bytes must be whole 16-byte pieces on 16-byte boundaries", row_bytes);
  if (rows == 0) return 0;
  const int chunks = row_bytes / 16;
  const long long total = (long long)rows * chunks;
  llg_launch(moe_gather_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const uint4*)x, token_of_row,
             (uint4*)out, rows, chunks);
  return llg_check_launch("moe_gather_rows");
}

// shared_scale: null, or [n_tokens]: the sum of the shared expert's partials is multiplied by it.
LLG_API int llg_moe_combine(const float* y, const int* row_of_pair, const float* weight, const float* shared, int n_shared,
                            long long shared_stride, const float* shared_scale, float* out, int n_tokens, int hidden, int top,
                            cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && hidden > 0 && top > 0, "moe_combine: bad sizes");
  LLG_REQUIRE(!shared || n_shared >= 1, "moe_combine: a shared expert's partials need at least one");
  if (n_tokens == 0) return 0;
  const bool vec = hidden % 4 == 0 && shared_stride % 4 == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)shared % 16) == 0 &&
                   ((uintptr_t)out % 16) == 0;
  if (vec) {
    const int threads = 128;
    dim3 grid(n_tokens, (hidden / 4 + threads - 1) / threads);
    llg_launch(moe_combine_vec4_kernel, grid, dim3(threads), 0, stream, y, row_of_pair, weight, shared, shared ? n_shared : 0,
               shared_stride, shared ? shared_scale : nullptr, out, hidden, top);
  } else {
    const int threads = hidden >= 1024 ? 256 : 128;
    llg_launch(moe_combine_kernel, dim3(n_tokens, 1), dim3(threads), 0, stream, y, row_of_pair, weight, shared,
               shared ? n_shared : 0, shared_stride, shared ? shared_scale : nullptr, out, hidden, top);
  }
  return llg_check_launch("moe_combine");
}
