// Kernels of latent attention (keys and values of all heads from one latent vector per token):
//
//   latent_prep : from the rows of the input product [q of all heads | latent | rotated key part] (float32 partial sums):
//                 the latent is RMS-normed with its weight, the rotated parts of every query head and the shared key part
//                 are rotated by the token's position (pairs (i, i + rot_dim/2), tables of cos and sin), and the results are
//                 written as the attention kernels read them: keys [latent | rotated part] and, where the caller keeps
//                 values apart, values [latent] for ONE key/value head (packed for a prompt step and/or into the cache
//                 pages), the queries' rotated parts behind
//                 the place where head_linear puts the unrotated parts' products, and the unrotated parts by themselves.
//   head_linear : y[n][h][:] = W_h x[n][h][:], a small product per (token, head) with one matrix per head; float32 sums.
//   sigmoid_gate: x *= sigmoid(columns of a product's float32 partial sums), in place (the gate on the concatenated heads).
//
// Statistics, angles' tables and sums are float32; inputs and outputs float32 or bfloat16.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

// Four neighbouring elements at once (the callers' hosts check sizes and addresses).
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const unsigned int*>(&lo);
  t.y = *reinterpret_cast<const unsigned int*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

// The queries' latent of token n: RMS norm over its cq_rank elements by a whole block (the latent is as long as a good
// part of the model's width).  Each thread adds the partial sums of its elements, four neighbours at a time where the
// host found that the sizes and addresses allow it (vec), once for the sum of squares and once more for the output.
template <typename OT, typename WT>
__device__ __forceinline__ void query_latent_norm(const LatentPrepArgs& a, int n, int vec) {
  __shared__ float scratch[32];
  const float* src = a.rows + (long long)n * a.row_width + a.cq_col;
  const WT* w = (const WT*)a.cq_norm_w;
  OT* o = (OT*)a.cq_out + (long long)n * a.cq_rank;
  float ss = 0.f;
  if (vec) {
    auto sum4 = [&](int d, float (&v)[4]) {
      load4(src + d, v);
      float t[4];
#pragma unroll 4
      for (int s = 1; s < a.n_partials; ++s) {
        load4(src + s * a.partial_stride + d, t);
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] += t[c];
      }
    };
    float v[4], ww[4];
    for (int d = threadIdx.x * 4; d < a.cq_rank; d += blockDim.x * 4) {
      sum4(d, v);
#pragma unroll
      for (int c = 0; c < 4; ++c) ss = fmaf(v[c], v[c], ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)a.cq_rank + a.norm_eps);
    for (int d = threadIdx.x * 4; d < a.cq_rank; d += blockDim.x * 4) {
      sum4(d, v);
      load4(w + d, ww);
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = v[c] * inv * ww[c];
      store4(o + d, v);
    }
    return;
  }
  auto summed = [&](int d) {
    float v = 0.f;
    for (int s = 0; s < a.n_partials; ++s) v += src[s * a.partial_stride + d];
    return v;
  };
  for (int d = threadIdx.x; d < a.cq_rank; d += blockDim.x) {
    const float v = summed(d);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)a.cq_rank + a.norm_eps);
  for (int d = threadIdx.x; d < a.cq_rank; d += blockDim.x) o[d] = from_f32<OT>(summed(d) * inv * to_f32(w[d]));
}

// One warp per unit of a token.  The units a launch has, in this order: the nh query heads (q_col >= 0), the latent with
// the shared key part (kv_col >= 0).  The blocks behind the units' (unit_blocks of them) take the queries' latent
// (cq_col >= 0), one block a token.
template <typename OT, typename WT>
__global__ void latent_prep_kernel(LatentPrepArgs a, int unit_blocks, int cq_vec) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= unit_blocks) {
    query_latent_norm<OT, WT>(a, (int)blockIdx.x - unit_blocks, cq_vec);
    return;
  }
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_units = a.q_col >= 0 ? a.nh : 0, kv_units = a.kv_col >= 0 ? 1 : 0;
  const int units = q_units + kv_units;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)a.n_tokens * units) return;
  const int n = (int)(item / units), u = (int)(item % units);
  const int qd = a.dim + a.rdim, kd = a.rank + a.rdim, half = a.rdim >> 1;
  const float* src = a.rows + (long long)n * a.row_width;
  const int pos = a.positions[n];
  const int p = pos < a.table_positions ? pos : a.table_positions - 1;        // bounded; the host checks the tables' reach
  const float* cs = a.cos_table ? a.cos_table + (long long)p * half : nullptr;
  const float* sn = a.sin_table ? a.sin_table + (long long)p * half : nullptr;
  // the two elements of pair i, counted from the rotated run's first element
  const int e1_step = a.pairing ? 2 : 1, e1_off = a.pairing ? 1 : half;
  auto summed = [&](long long col) {
    float v = 0.f;
    for (int s = 0; s < a.n_partials; ++s) v += src[s * a.partial_stride + col];
    return v;
  };
  if (u < q_units) {
    const long long col = a.q_col + (long long)u * qd;
    OT* qp = (OT*)a.q_plain + ((long long)n * a.nh + u) * a.dim;
    for (int d = lane; d < a.dim; d += 32) qp[d] = from_f32<OT>(summed(col + d));
    OT* qo = (OT*)a.q_out + ((long long)n * a.nh + u) * kd + a.rank;
    for (int i = lane; i < half; i += 32) {
      const int e0 = i * e1_step, e1 = e0 + e1_off;
      const float x0 = summed(col + a.dim + e0), x1 = summed(col + a.dim + e1);
      qo[e0] = from_f32<OT>(x0 * cs[i] - x1 * sn[i]);
      qo[e1] = from_f32<OT>(x1 * cs[i] + x0 * sn[i]);
    }
    return;
  }
  const WT* w = (const WT*)a.c_norm_w;
  // the latent: RMS norm over its kv_rank elements
  const long long col = a.kv_col;
  float ss = 0.f;
  for (int d = lane; d < a.rank; d += 32) {
    const float v = summed(col + d);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.norm_eps);
  OT* kn = a.k_new ? (OT*)a.k_new + (long long)n * kd : nullptr;
  OT* vn = a.v_new ? (OT*)a.v_new + (long long)n * a.rank : nullptr;
  OT *kp = nullptr, *vp = nullptr;
  if (a.k_pages) {
    const int slot = a.slots[a.seq_of_token[n]];
    const long long r = kv_row(a.page_table, a.table_width, a.ring_pages, slot, pos, 0, 1);
    kp = (OT*)a.k_pages + r * kd;
    vp = a.v_pages ? (OT*)a.v_pages + r * a.rank : nullptr;
  }
  for (int d = lane; d < a.rank; d += 32) {
    const OT c = from_f32<OT>(summed(col + d) * inv * to_f32(w[d]));
    if (kn) kn[d] = c;
    if (vn) vn[d] = c;
    if (kp) kp[d] = c;
    if (vp) vp[d] = c;
  }
  for (int i = lane; i < half; i += 32) {
    const int e0 = i * e1_step, e1 = e0 + e1_off;
    const float x0 = summed(col + a.rank + e0), x1 = summed(col + a.rank + e1);
    const OT r0 = from_f32<OT>(x0 * cs[i] - x1 * sn[i]), r1 = from_f32<OT>(x1 * cs[i] + x0 * sn[i]);
    if (kn) { kn[a.rank + e0] = r0; kn[a.rank + e1] = r1; }
    if (kp) { kp[a.rank + e0] = r0; kp[a.rank + e1] = r1; }
  }
}

// x[n][j] *= sigmoid(sum of the partials gate[.][n][col0 + j] + bias[j]): a gate whose arguments are columns of another
// product's float32 partial sums, applied in place.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, int n_partials, long long partial_stride,
                                    int gate_width, int col0, const float* __restrict__ bias, long long total, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long n = i / width;
  const int j = (int)(i % width);
  const float* g = gate + n * gate_width + col0 + j;
  float z = bias ? bias[j] : 0.f;
  for (int s = 0; s < n_partials; ++s) z += g[s * partial_stride];
  x[i] = from_f32<T>(to_f32(x[i]) / (1.0f + expf(-z)));
}

// The same, four neighbouring elements of a row per thread (the host checks that rows, columns and addresses allow it).
template <typename T>
__global__ void sigmoid_gate4_kernel(T* __restrict__ x, const float* __restrict__ gate, int n_partials, long long partial_stride,
                                     int gate_width, int col0, const float* __restrict__ bias, long long total, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= total) return;
  const long long n = i / width;
  const int j = (int)(i % width);
  const float* g = gate + n * gate_width + col0 + j;
  float z[4], t[4], v[4];
  load4(g, z);
#pragma unroll 4
  for (int s = 1; s < n_partials; ++s) {
    load4(g + s * partial_stride, t);
#pragma unroll
    for (int c = 0; c < 4; ++c) z[c] += t[c];
  }
  if (bias) {
    load4(bias + j, t);
#pragma unroll
    for (int c = 0; c < 4; ++c) z[c] += t[c];
  }
  load4(x + i, v);
#pragma unroll
  for (int c = 0; c < 4; ++c) v[c] = v[c] / (1.0f + expf(-z[c]));
  store4(x + i, v);
}

// y[n][h][o] = sum_k w[h][o][k] x[n][h][k].  A block takes TN tokens of one head and TO outputs; x's tile lies in shared
// memory as float32, a thread owns one output column for TN / (threads / TO) tokens... kept simple: thread (to, tn)
// computes y for output to0 + to and tokens tn, tn + TY, ...; w rows are read once per block through shared memory.
constexpr int HL_TN = 32, HL_TO = 32, HL_TK = 32;

template <typename XT, typename WT, typename YT>
__global__ void __launch_bounds__(256) head_linear_kernel(HeadLinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[HL_TN][HL_TK + 1];
  __shared__ float ws[HL_TO][HL_TK + 1];
  const int h = blockIdx.z;
  const int n0 = blockIdx.x * HL_TN, o0 = blockIdx.y * HL_TO;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // tx: output within the tile, ty: 8 token groups
  const XT* x = (const XT*)a.x;
  const WT* w = (const WT*)a.w + (long long)h * a.n_out * a.n_in;
  float acc[HL_TN / 8];
#pragma unroll
  for (int i = 0; i < HL_TN / 8; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < a.n_in; k0 += HL_TK) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < HL_TN * HL_TK; idx += 256) {
      const int r = idx / HL_TK, c = idx % HL_TK;
      const int n = n0 + r, k = k0 + c;
      xs[r][c] = (n < a.n_tokens && k < a.n_in) ? to_f32(x[(long long)n * a.x_token_stride + (long long)h * a.x_head_stride + k]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < HL_TO * HL_TK; idx += 256) {
      const int r = idx / HL_TK, c = idx % HL_TK;
      const int o = o0 + r, k = k0 + c;
      ws[r][c] = (o < a.n_out && k < a.n_in) ? to_f32(w[(long long)o * a.n_in + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_TK; ++k) {
      const float wv = ws[tx][k];
#pragma unroll
      for (int i = 0; i < HL_TN / 8; ++i) acc[i] = fmaf(xs[ty + 8 * i][k], wv, acc[i]);
    }
  }
  YT* y = (YT*)a.y;
  const int o = o0 + tx;
  if (o < a.n_out) {
#pragma unroll
    for (int i = 0; i < HL_TN / 8; ++i) {
      const int n = n0 + ty + 8 * i;
      if (n < a.n_tokens) y[(long long)n * a.y_token_stride + (long long)h * a.y_head_stride + o] = from_f32<YT>(acc[i]);
    }
  }
}

}  // namespace

LLG_API int llg_latent_prep(const LatentPrepArgs* args, int out_dtype, cudaStream_t stream) {
  const LatentPrepArgs& a = *args;
  LLG_REQUIRE(a.n_tokens >= 0 && a.nh > 0 && a.dim > 0 && a.rank > 0 && a.rdim >= 0 && a.rdim % 2 == 0, "latent_prep: bad sizes");
  LLG_REQUIRE(a.n_partials >= 1, "latent_prep: n_partials must be >= 1");
  LLG_REQUIRE(a.pairing == 0 || a.pairing == 1, "latent_prep: pairing %d is not known", a.pairing);
  LLG_REQUIRE(a.q_col < 0 || (a.q_plain && a.q_out && a.q_col + (long long)a.nh * (a.dim + a.rdim) <= a.row_width),
              "latent_prep: the queries' columns need their outputs and must lie inside the row");
  LLG_REQUIRE(a.kv_col < 0 || a.kv_col + a.rank + a.rdim <= a.row_width, "latent_prep: the latent's columns must lie inside the row");
  LLG_REQUIRE(a.cq_col < 0 || (a.cq_rank > 0 && a.cq_norm_w && a.cq_out && a.cq_col + a.cq_rank <= a.row_width),
              "latent_prep: the queries' latent needs its size, weight and output and must lie inside the row");
  LLG_REQUIRE(a.kv_col >= 0 || (!a.k_new && !a.k_pages), "latent_prep: keys are written where the latent is given");
  LLG_REQUIRE(a.rdim == 0 || (a.cos_table && a.sin_table && a.table_positions > 0), "latent_prep: rotated elements need the tables");
  LLG_REQUIRE(!a.k_pages || (a.page_table && a.slots && a.seq_of_token && a.ring_pages > 0),
              "latent_prep: a cache write needs page_table, slots and seq_of_token");
  LLG_REQUIRE((!a.v_new || a.k_new) && (!a.v_pages || a.k_pages), "latent_prep: values are written beside keys only");
  if (a.n_tokens == 0) return 0;
  const int warps = 4;
  const long long items = (long long)a.n_tokens * ((a.q_col >= 0 ? a.nh : 0) + (a.kv_col >= 0 ? 1 : 0));
  const int unit_blocks = (int)((items + warps - 1) / warps);
  const int cq_vec = a.cq_col >= 0 && a.cq_col % 4 == 0 && a.cq_rank % 4 == 0 && a.row_width % 4 == 0 && a.partial_stride % 4 == 0 &&
             (size_t)a.rows % 16 == 0 && (size_t)a.cq_norm_w % 16 == 0 && (size_t)a.cq_out % 16 == 0;
  const long long blocks = (long long)unit_blocks + (a.cq_col >= 0 ? a.n_tokens : 0);
  if (blocks == 0) return 0;
  LLG_REQUIRE(blocks < 2147483647LL, "latent_prep: too many blocks");
  const unsigned grid = (unsigned)blocks;
  const bool wb = a.w_dtype == LLG_BF16;
  if (out_dtype == LLG_F32) {
    if (wb) llg_launch(latent_prep_kernel<float, __nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, a, unit_blocks, cq_vec);
    else llg_launch(latent_prep_kernel<float, float>, dim3(grid), dim3(warps * 32), 0, stream, a, unit_blocks, cq_vec);
  } else if (out_dtype == LLG_BF16) {
    if (wb) llg_launch(latent_prep_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, a, unit_blocks, cq_vec);
    else llg_launch(latent_prep_kernel<__nv_bfloat16, float>, dim3(grid), dim3(warps * 32), 0, stream, a, unit_blocks, cq_vec);
  } else {
    return llg_fail("latent_prep: unknown output dtype %d", out_dtype);
  }
  return llg_check_launch("latent_prep");
}

// y_dtype: the outputs' type; float32 outputs go with inputs of either type (the sums are float32 anyway).
LLG_API int llg_head_linear(const HeadLinearArgs* args, int dtype, int y_dtype, cudaStream_t stream) {
  const HeadLinearArgs& a = *args;
  LLG_REQUIRE(a.n_tokens >= 0 && a.nh > 0 && a.n_in > 0 && a.n_out > 0, "head_linear: bad sizes");
  LLG_REQUIRE(a.nh <= 65535, "head_linear: too many heads");
  if (a.n_tokens == 0) return 0;
  dim3 grid((a.n_tokens + HL_TN - 1) / HL_TN, (a.n_out + HL_TO - 1) / HL_TO, a.nh);
  if (dtype == LLG_F32 && y_dtype == LLG_F32) llg_launch(head_linear_kernel<float, float, float>, grid, dim3(256), 0, stream, a);
  else if (dtype == LLG_BF16 && y_dtype == LLG_BF16)
    llg_launch(head_linear_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream, a);
  else if (dtype == LLG_BF16 && y_dtype == LLG_F32)
    llg_launch(head_linear_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, dim3(256), 0, stream, a);
  else return llg_fail("head_linear: unknown types %d -> %d", dtype, y_dtype);
  return llg_check_launch("head_linear");
}

LLG_API int llg_sigmoid_gate(void* x, int dtype, const float* gate, int n_partials, long long partial_stride, int gate_width,
                             int col0, const float* bias, int n_tokens, int width, cudaStream_t stream) {
  LLG_REQUIRE(n_tokens >= 0 && width > 0 && n_partials >= 1 && col0 >= 0 && col0 + width <= gate_width,
              "sigmoid_gate: bad sizes (width %d at column %d of %d)", width, col0, gate_width);
  if (n_tokens == 0) return 0;
  const long long total = (long long)n_tokens * width;
  const bool vec = width % 4 == 0 && col0 % 4 == 0 && gate_width % 4 == 0 && partial_stride % 4 == 0 && (size_t)x % 16 == 0 &&
                   (size_t)gate % 16 == 0 && (size_t)bias % 16 == 0;
  const unsigned grid = (unsigned)(((vec ? total / 4 : total) + 255) / 256);
#define GATE(T)                                                                                                          \
  do {                                                                                                                   \
    if (vec) llg_launch(sigmoid_gate4_kernel<T>, dim3(grid), dim3(256), 0, stream, (T*)x, gate, n_partials, partial_stride, \
                        gate_width, col0, bias, total, width);                                                           \
    else llg_launch(sigmoid_gate_kernel<T>, dim3(grid), dim3(256), 0, stream, (T*)x, gate, n_partials, partial_stride,   \
                    gate_width, col0, bias, total, width);                                                               \
  } while (0)
  if (dtype == LLG_F32) GATE(float);
  else if (dtype == LLG_BF16) GATE(__nv_bfloat16);
#undef GATE
  else return llg_fail("sigmoid_gate: unknown dtype %d", dtype);
  return llg_check_launch("sigmoid_gate");
}
