// Recurrent mixers' scans (argument blocks in kernel_args.h).
//
//   mingru_scan : S_t = (1 - z_t) S_{t-1} + z_t c_t per channel along every sequence of a step, from the state the cache
//                 holds; writes S_t * silu(g_t) and leaves the last state.  A thread owns one channel of one sequence (or
//                 of one piece of it) and walks the tokens in order; neighbouring threads read neighbouring columns.
//                 Long prompts are cut into pieces that are scanned side by side and joined (MinGruArgs).
//
// Gates, candidates, the state and every sum are float32 whatever the output type.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_mingru_piece() { return LLG_MINGRU_PIECE; }

namespace {

// 1 / (1 + exp(-v)) with the correctly rounded reciprocal: the same float as the division gives, in fewer instructions
__device__ __forceinline__ float sigmoid_f(float v) { return __frcp_rn(1.0f + expf(-v)); }

constexpr int SCAN_BATCH = 8;      // tokens (or pieces) whose loads are issued together, ahead of the arithmetic and the stores

// MODE 0: the whole sequence from state[slot], outputs and the last state written (no carry).
// MODE 1: a piece from zero; writes (product of 1 - z, state reached) to carry.
// MODE 2: a piece from carry's starting state; writes outputs.
// The arguments of SCAN_BATCH tokens are summed from the partials into registers first: the loads of a batch do not wait
// for one another nor for the stores of the tokens before them, which is what bounds a walk along a sequence.
template <typename OT, int MODE>
__global__ void __launch_bounds__(128) mingru_scan_kernel(MinGruArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int piece = blockIdx.y, b = blockIdx.z;
  if (ch >= a.size) return;
  const int t_begin = a.cu_tokens[b], t_end = a.cu_tokens[b + 1];
  int lo = t_begin, hi = t_end;
  if (MODE != 0) {
    // the last piece takes whatever is left, so no token is lost where the host counted too few pieces
    lo = t_begin + piece * LLG_MINGRU_PIECE;
    if (lo > t_end) lo = t_end;
    hi = (piece == a.pieces - 1 || lo + LLG_MINGRU_PIECE > t_end) ? t_end : lo + LLG_MINGRU_PIECE;
  }
  float* cr = MODE != 0 ? a.carry + (((long long)b * a.pieces + piece) * 2) * a.size + ch : nullptr;
  const float bz = a.bias[ch], bu = a.bias[a.size + ch];
  float S = 0.f, A = 1.f;
  if (MODE == 0) S = a.state[(long long)a.slots[b] * a.size + ch];
  if (MODE == 2) {
    if (lo >= hi) return;
    S = cr[a.size];
  }
  OT* out = (OT*)a.out;
  const long long row = 3LL * a.size;
  for (int n0 = lo; n0 < hi; n0 += SCAN_BATCH) {
    float z[SCAN_BATCH], u[SCAN_BATCH], g[SCAN_BATCH];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) { z[k] = bz; u[k] = bu; g[k] = 0.f; }
    for (int s = 0; s < a.n_partials; ++s) {
      const float* p = a.rows + s * a.partial_stride + n0 * row + ch;
#pragma unroll
      for (int k = 0; k < SCAN_BATCH; ++k) {
        if (n0 + k < hi) {
          z[k] += p[k * row];
          u[k] += p[k * row + a.size];
          if (MODE != 1) g[k] += p[k * row + 2 * a.size];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (n0 + k < hi) {
        const float zt = sigmoid_f(z[k]);
        const float ct = u[k] >= 0.f ? u[k] + 0.5f : sigmoid_f(u[k]);
        S = (1.0f - zt) * S + zt * ct;
        if (MODE == 1) A *= 1.0f - zt;
        else out[(long long)(n0 + k) * a.size + ch] = from_f32<OT>(S * (g[k] * sigmoid_f(g[k])));
      }
    }
  }
  if (MODE == 0) a.state[(long long)a.slots[b] * a.size + ch] = S;
  if (MODE == 1) {
    cr[0] = A;
    cr[a.size] = S;
  }
}

// Walks a sequence's pieces: piece p starts from what the pieces before it make of the sequence's state.
__global__ void __launch_bounds__(128) mingru_join_kernel(MinGruArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (ch >= a.size) return;
  float* st = a.state + (long long)a.slots[b] * a.size + ch;
  float S = *st;
  float* cr = a.carry + ((long long)b * a.pieces * 2) * a.size + ch;
  const long long step = 2LL * a.size;
  for (int p0 = 0; p0 < a.pieces; p0 += SCAN_BATCH, cr += SCAN_BATCH * step) {
    float A[SCAN_BATCH], B[SCAN_BATCH];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (p0 + k < a.pieces) {
        A[k] = cr[k * step];
        B[k] = cr[k * step + a.size];
      }
    }
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (p0 + k < a.pieces) {
        cr[k * step + a.size] = S;
        S = A[k] * S + B[k];
      }
    }
  }
  *st = S;
}

template <typename OT>
int mingru_launch(const MinGruArgs& a, cudaStream_t stream) {
  const unsigned cb = (unsigned)((a.size + 127) / 128);
  if (!a.carry) {
    llg_launch(mingru_scan_kernel<OT, 0>, dim3(cb, 1, a.n_seqs), dim3(128), 0, stream, a);
    return llg_check_launch("mingru_scan");
  }
  llg_launch(mingru_scan_kernel<OT, 1>, dim3(cb, a.pieces, a.n_seqs), dim3(128), 0, stream, a);
  llg_launch(mingru_join_kernel, dim3(cb, a.n_seqs), dim3(128), 0, stream, a);
  llg_launch(mingru_scan_kernel<OT, 2>, dim3(cb, a.pieces, a.n_seqs), dim3(128), 0, stream, a);
  return llg_check_launch("mingru_scan (pieces)");
}

}  // namespace

// max_count: the most tokens a sequence of the step brings (the host knows it; the kernels read cu_tokens).
LLG_API int llg_mingru_scan(const MinGruArgs* args, int max_count, cudaStream_t stream) {
  const MinGruArgs& a = *args;
  LLG_REQUIRE(a.n_seqs >= 0 && a.n_tokens >= 0 && a.size > 0 && a.n_partials >= 1, "mingru_scan: bad sizes");
  LLG_REQUIRE(a.n_seqs <= 65535, "mingru_scan: %d sequences in a step (at most 65535)", a.n_seqs);
  if (a.carry)
    LLG_REQUIRE(a.pieces >= 1 && a.pieces <= 65535 && (long long)a.pieces * LLG_MINGRU_PIECE >= max_count,
                "mingru_scan: %d pieces of %d tokens do not hold a sequence of %d", a.pieces, LLG_MINGRU_PIECE, max_count);
  if (a.n_seqs == 0 || a.n_tokens == 0) return 0;
  if (a.out_dtype == LLG_F32) return mingru_launch<float>(a, stream);
  if (a.out_dtype == LLG_BF16) return mingru_launch<__nv_bfloat16>(a, stream);
  return llg_fail("mingru_scan: unknown output type %d", a.out_dtype);
}
