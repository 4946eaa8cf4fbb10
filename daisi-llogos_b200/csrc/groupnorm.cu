// RMS norm in groups fused with the residual add, the add optionally through a sigmoid gate and a norm of its own; see
// GroupNormArgs in kernel_args.h.  One block per output row; the row lies in shared memory as float32 between the passes
// (branch and gate, the branch's own norm, the add, the norm of the sum).  A group's sum of squares belongs to a team of
// warps (the block's warps divided among the groups; with more groups than warps the teams take them in rounds): every
// warp adds its share by shuffles, the team's sums are added in a fixed order, and the same warps then scale what they
// summed.  So a row's result does not depend on what else the launch holds.  Where the sizes allow (VEC 4: the group size
// a multiple of four, 16-byte aligned operands) every access moves four elements.  The residual, the gate, every sum
// and every statistic are float32.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_norm_max_groups() { return LLG_NORM_MAX_GROUPS; }

namespace {

template <int VEC> struct Pack { float v[VEC]; };

template <int VEC> __device__ __forceinline__ Pack<VEC> load_f32(const float* p) {
  Pack<VEC> r;
  if (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[VEC > 1 ? 1 : 0] = t.y; r.v[VEC > 2 ? 2 : 0] = t.z; r.v[VEC > 3 ? 3 : 0] = t.w; }
  else r.v[0] = *p;
  return r;
}
template <int VEC> __device__ __forceinline__ Pack<VEC> load_w(const float* p) { return load_f32<VEC>(p); }
template <int VEC> __device__ __forceinline__ Pack<VEC> load_w(const __nv_bfloat16* p) {
  Pack<VEC> r;
  if (VEC == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    r.v[0] = __uint_as_float(t.x << 16); r.v[VEC > 1 ? 1 : 0] = __uint_as_float(t.x & 0xffff0000u);
    r.v[VEC > 2 ? 2 : 0] = __uint_as_float(t.y << 16); r.v[VEC > 3 ? 3 : 0] = __uint_as_float(t.y & 0xffff0000u);
  } else r.v[0] = __bfloat162float(*p);
  return r;
}
template <int VEC> __device__ __forceinline__ void store(float* p, const Pack<VEC>& r) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[VEC > 1 ? 1 : 0], r.v[VEC > 2 ? 2 : 0], r.v[VEC > 3 ? 3 : 0]);
  else *p = r.v[0];
}
template <int VEC> __device__ __forceinline__ void store(__nv_bfloat16* p, const Pack<VEC>& r) {
  if (VEC == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[VEC > 1 ? 1 : 0]), hi = __floats2bfloat162_rn(r.v[VEC > 2 ? 2 : 0], r.v[VEC > 3 ? 3 : 0]);
    uint2 t;
    t.x = *reinterpret_cast<const unsigned int*>(&lo);
    t.y = *reinterpret_cast<const unsigned int*>(&hi);
    *reinterpret_cast<uint2*>(p) = t;
  } else *p = __float2bfloat16_rn(r.v[0]);
}

// row[i] <- row[i] / sqrt(mean of its group's squares + eps) * w[i], or, with `out`, the same written there instead.
// Called by every thread of the block; `part` holds one float per warp.
template <int VEC, typename WT, typename OT>
__device__ __forceinline__ void group_rms(float* row, int hidden, int groups, float eps, const WT* w, OT* out, float* part) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int gs = hidden / groups;
  const int team_warps = nwarps / groups > 0 ? nwarps / groups : 1;      // warps per group
  const int teams = nwarps / team_warps;                                  // groups in flight
  const int team = warp / team_warps, rank = warp - team * team_warps;
  for (int g0 = 0; g0 < groups; g0 += teams) {
    const int g = g0 + team;
    const bool on = team < teams && g < groups;
    float* p = row + (long long)(on ? g : 0) * gs;
    if (on) {
      float ss = 0.f;
      for (int i = (rank * 32 + lane) * VEC; i < gs; i += team_warps * 32 * VEC) {
        const Pack<VEC> v = load_f32<VEC>(p + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) ss = fmaf(v.v[c], v.v[c], ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) part[warp] = ss;
    }
    __syncthreads();
    if (on) {
      float ss = 0.f;
      for (int t = 0; t < team_warps; ++t) ss += part[team * team_warps + t];
      const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
      const WT* wg = w + (long long)g * gs;
      for (int i = (rank * 32 + lane) * VEC; i < gs; i += team_warps * 32 * VEC) {
        Pack<VEC> v = load_f32<VEC>(p + i);
        const Pack<VEC> ww = load_w<VEC>(wg + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) v.v[c] = v.v[c] * inv * ww.v[c];
        if (out) store<VEC>(out + (long long)g * gs + i, v);
        else store<VEC>(p + i, v);
      }
    }
    __syncthreads();
  }
}

template <int VEC, typename OT, typename WT>
__global__ void __launch_bounds__(1024) gated_add_group_rmsnorm_kernel(GroupNormArgs a, int early_residual) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float row[];
  __shared__ float part[32];
  const int j = blockIdx.x;
  const int r = a.rows ? a.rows[j] : j;
  const int hidden = a.hidden;
  float* res = a.residual + (long long)r * hidden;
  // early_residual: a second row of shared memory takes the residual while the branch is read, so that the add after the
  // branch's norm does not wait for memory once more
  float* res_row = early_residual ? row + hidden : nullptr;
  if (a.branch) {
    const float* bp = a.branch + (long long)r * hidden;
    const float* gp = a.gate ? a.gate + (long long)r * hidden : nullptr;
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
      if (res_row) store<VEC>(res_row + i, load_f32<VEC>(res + i));
      Pack<VEC> y = load_f32<VEC>(bp + i);
#pragma unroll 4
      for (int s = 1; s < a.n_partials; ++s) {
        const Pack<VEC> t = load_f32<VEC>(bp + s * a.partial_stride + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) y.v[c] += t.v[c];
      }
      if (gp) {
        Pack<VEC> z = load_f32<VEC>(gp + i);
#pragma unroll 4
        for (int s = 1; s < a.gate_partials; ++s) {
          const Pack<VEC> t = load_f32<VEC>(gp + s * a.partial_stride + i);
#pragma unroll
          for (int c = 0; c < VEC; ++c) z.v[c] += t.v[c];
        }
        if (a.gate_bias) {
          const Pack<VEC> b = load_f32<VEC>(a.gate_bias + i);
#pragma unroll
          for (int c = 0; c < VEC; ++c) z.v[c] += b.v[c];
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) y.v[c] = y.v[c] / (1.0f + expf(-z.v[c]));
      }
      store<VEC>(row + i, y);
    }
    __syncthreads();
    if (a.post_w) group_rms<VEC, WT, float>(row, hidden, a.post_groups, a.post_eps, (const WT*)a.post_w, nullptr, part);
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
      Pack<VEC> v = load_f32<VEC>(res_row ? res_row + i : res + i);
      const Pack<VEC> y = load_f32<VEC>(row + i);
#pragma unroll
      for (int c = 0; c < VEC; ++c) v.v[c] += y.v[c];
      store<VEC>(res + i, v);
      store<VEC>(row + i, v);
    }
  } else {
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) store<VEC>(row + i, load_f32<VEC>(res + i));
  }
  __syncthreads();
  group_rms<VEC, WT, OT>(row, hidden, a.groups, a.eps, (const WT*)a.weight, (OT*)a.out + (long long)j * hidden, part);
}

}  // namespace

LLG_API int llg_gated_add_group_rmsnorm(const GroupNormArgs* args, cudaStream_t stream) {
  const GroupNormArgs& a = *args;
  LLG_REQUIRE(a.n_out >= 0 && a.hidden > 0, "group_rmsnorm: bad sizes n_out=%d hidden=%d", a.n_out, a.hidden);
  LLG_REQUIRE(a.eps > 0.f && a.groups >= 1 && a.groups <= LLG_NORM_MAX_GROUPS && a.hidden % a.groups == 0,
              "group_rmsnorm: %d elements in %d groups (at most %d), eps %g", a.hidden, a.groups, LLG_NORM_MAX_GROUPS, a.eps);
  LLG_REQUIRE(!a.branch || a.n_partials >= 1, "group_rmsnorm: a branch needs at least one partial");
  LLG_REQUIRE(a.branch || (!a.gate && !a.post_w), "group_rmsnorm: a gate or a norm of the branch needs the branch");
  LLG_REQUIRE(!a.gate || a.gate_partials >= 1, "group_rmsnorm: a gate needs at least one partial");
  LLG_REQUIRE(!a.post_w || (a.post_eps > 0.f && a.post_groups >= 1 && a.post_groups <= LLG_NORM_MAX_GROUPS &&
                            a.hidden % a.post_groups == 0),
              "group_rmsnorm: the branch's norm has %d groups over %d elements, eps %g", a.post_groups, a.hidden, a.post_eps);
  if (a.n_out == 0) return 0;
  // Four elements per access where every group is a multiple of four long and the operands are 16-byte aligned (the
  // weights and a bfloat16 output 8-byte); one access per thread up to 4096 elements a row, so that a step of few rows
  // has its loads in flight together.
  const int gs = a.hidden / a.groups, post_gs = a.post_w ? a.hidden / a.post_groups : 4;
  auto aligned = [](const void* p, size_t n) { return p == nullptr || ((size_t)p % n) == 0; };
  const bool vec = gs % 4 == 0 && post_gs % 4 == 0 && a.partial_stride % 4 == 0 && aligned(a.residual, 16) && aligned(a.branch, 16) &&
                   aligned(a.gate, 16) && aligned(a.gate_bias, 16) && aligned(a.post_w, 16) && aligned(a.weight, 16) && aligned(a.out, 16);
  const int per_thread = vec ? 4 : 1;
  int threads = ((a.hidden + per_thread - 1) / per_thread + 31) / 32 * 32;
  // many rows: blocks of 512 threads at most, so that an SM holds several rows at different stages
  const int most = a.n_out > 2 * llg_sm_count() ? 512 : 1024;
  threads = threads < 128 ? 128 : (threads > most ? most : threads);
  LLG_REQUIRE((size_t)a.hidden * sizeof(float) <= 200 * 1024, "group_rmsnorm: rows of %d elements do not fit shared memory", a.hidden);
  const int early_residual = a.branch && (size_t)a.hidden * sizeof(float) <= 48 * 1024;
  const size_t smem = (size_t)a.hidden * sizeof(float) * (early_residual ? 2 : 1);
#define LAUNCH_V(V, OT, WT)                                                                                     \
  do {                                                                                                          \
    auto k = gated_add_group_rmsnorm_kernel<V, OT, WT>;                                                         \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      if (e != cudaSuccess) return llg_fail("group_rmsnorm: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                           \
    llg_launch(k, dim3(a.n_out), dim3(threads), smem, stream, a, early_residual);                                              \
  } while (0)
#define LAUNCH(OT, WT)                      \
  do {                                      \
    if (vec) LAUNCH_V(4, OT, WT);           \
    else LAUNCH_V(1, OT, WT);               \
  } while (0)
  if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_F32) LAUNCH(float, float);
  else if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return llg_fail("group_rmsnorm: unknown dtypes out=%d weight=%d", a.out_dtype, a.w_dtype);
#undef LAUNCH
#undef LAUNCH_V
  return llg_check_launch("group_rmsnorm");
}
