// RMS norm in groups fused with the residual add, the add optionally through a sigmoid gate and a norm of its own; see
// GroupNormArgs in kernel_args.h.  One block per output row; the row lies in shared memory as float32 between the passes
// (branch and gate, the branch's own norm, the add, the norm of the sum).  A group's sum of squares is one warp's: the
// warp's lanes walk the group's elements and the lanes' sums are added by shuffles, so a row's result does not depend on
// what else the launch holds.  The residual, the gate, every sum and every statistic are float32.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_norm_max_groups() { return LLG_NORM_MAX_GROUPS; }

namespace {

// row[i] <- row[i] / sqrt(mean of its group's squares + eps) * w[i], or, with `out`, the same written there instead
template <typename WT, typename OT>
__device__ __forceinline__ void group_rms(float* row, int hidden, int groups, float eps, const WT* w, OT* out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int gs = hidden / groups;
  for (int g = warp; g < groups; g += nwarps) {
    float* p = row + (long long)g * gs;
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
    const WT* wg = w + (long long)g * gs;
    if (out) {
      OT* o = out + (long long)g * gs;
      for (int i = lane; i < gs; i += 32) o[i] = from_f32<OT>(p[i] * inv * to_f32(wg[i]));
    } else {
      for (int i = lane; i < gs; i += 32) p[i] = p[i] * inv * to_f32(wg[i]);
    }
  }
}

template <typename OT, typename WT>
__global__ void gated_add_group_rmsnorm_kernel(GroupNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  const int j = blockIdx.x;
  const int r = a.rows ? a.rows[j] : j;
  const int hidden = a.hidden;
  float* res = a.residual + (long long)r * hidden;
  if (a.branch) {
    const float* bp = a.branch + (long long)r * hidden;
    const float* gp = a.gate ? a.gate + (long long)r * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float y = 0.f;
      for (int s = 0; s < a.n_partials; ++s) y += bp[s * a.partial_stride + i];
      if (gp) {
        float z = a.gate_bias ? a.gate_bias[i] : 0.f;
        for (int s = 0; s < a.gate_partials; ++s) z += gp[s * a.partial_stride + i];
        y = y / (1.0f + expf(-z));
      }
      row[i] = y;
    }
    __syncthreads();
    if (a.post_w) {
      group_rms<WT, float>(row, hidden, a.post_groups, a.post_eps, (const WT*)a.post_w, nullptr);
      __syncthreads();
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = res[i] + row[i];
      res[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row[i] = res[i];
  }
  __syncthreads();
  group_rms<WT, OT>(row, hidden, a.groups, a.eps, (const WT*)a.weight, (OT*)a.out + (long long)j * hidden);
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
  const int threads = a.hidden >= 4096 ? 512 : (a.hidden >= 1024 ? 256 : 128);
  const size_t smem = (size_t)a.hidden * sizeof(float);
  LLG_REQUIRE(smem <= 200 * 1024, "group_rmsnorm: rows of %d elements do not fit shared memory", a.hidden);
#define LAUNCH(OT, WT)                                                                                          \
  do {                                                                                                          \
    auto k = gated_add_group_rmsnorm_kernel<OT, WT>;                                                            \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      if (e != cudaSuccess) return llg_fail("group_rmsnorm: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                           \
    llg_launch(k, dim3(a.n_out), dim3(threads), smem, stream, a);                                               \
  } while (0)
  if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_F32) LAUNCH(float, float);
  else if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return llg_fail("group_rmsnorm: unknown dtypes out=%d weight=%d", a.out_dtype, a.w_dtype);
#undef LAUNCH
  return llg_check_launch("group_rmsnorm");
}
