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

// ---- short causal convolutions, the real-gated linear recurrent unit, retention -----------------------------------------
//
//   causal_conv : a thread owns one (token, channel).  The tokens of a sequence whose taps reach back before the step
//                 (the first taps - 1 of its step tokens) are all done by the thread of the sequence's first token, which
//                 reads the slot's state first and writes the new state last: nobody else touches that state, so nothing
//                 of a step can read what the same step has already replaced.
//   rglru_scan  : the minGRU scan's three modes with the unit's own gates (RgLruArgs); pieces are joined by
//                 mingru_join_kernel, which only walks (factor, offset) pairs.
//   retention   : a block owns one (sequence or piece, head) with the head's state [dim][vdim] in shared memory and walks
//                 the tokens in order: S <- decay S + k v^T, o = S^T q, then the head's unit norm and the silu gate.
//                 Rotation of q and k happens here, in float32, from the product's float32 sums.

namespace {

template <typename O2>
__global__ void __launch_bounds__(128) causal_conv_kernel(ConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int K = a.taps;
  const int b = a.seq_of_token[n];
  const int t0 = a.cu_tokens[b], count = a.cu_tokens[b + 1] - t0;
  const int p = n - t0;
  if (p > 0 && p < K - 1) return;                  // done by the thread of the sequence's first step token
  const float ib = a.in_bias ? a.in_bias[c] : 0.f, ob = a.bias ? a.bias[c] : 0.f;
  float w[LLG_CONV_MAX_TAPS];
  for (int j = 0; j < K; ++j) w[j] = a.weight[(long long)c * K + j];
  auto input = [&](int q) {                        // the input at step token q of this sequence
    const float* r = a.rows + (long long)(t0 + q) * a.row_width + a.col0 + c;
    float v = r[0];
    for (int s = 1; s < a.n_partials; ++s) v += r[s * a.partial_stride];
    return v + ib;
  };
  O2* out2 = (O2*)a.out2;
  if (p >= K - 1) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc = fmaf(w[j], input(p - (K - 1) + j), acc);
    acc += ob;
    a.out[(long long)n * a.channels + c] = acc;
    if (out2) out2[(long long)n * a.channels + c] = from_f32<O2>(acc);
    return;
  }
  // p == 0 and K >= 2: vals[0 .. K-2] the inputs before the step, vals[K-1 + q] the step's first ones
  float vals[2 * LLG_CONV_MAX_TAPS];
  float* st = a.state + (long long)a.slots[b] * (K - 1) * a.channels + c;
  const int lb = a.len_before[b];
  for (int s = 0; s < K - 1; ++s) vals[s] = (lb - (K - 1) + s >= 0) ? st[(long long)s * a.channels] : 0.f;
  const int m = count < K - 1 ? count : K - 1;
  for (int q = 0; q < m; ++q) vals[K - 1 + q] = input(q);
  for (int q = 0; q < m; ++q) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc = fmaf(w[j], vals[q + j], acc);
    acc += ob;
    a.out[(long long)(t0 + q) * a.channels + c] = acc;
    if (out2) out2[(long long)(t0 + q) * a.channels + c] = from_f32<O2>(acc);
  }
  float fresh[LLG_CONV_MAX_TAPS];
  for (int s = 0; s < K - 1; ++s) {
    const int q = count - (K - 1) + s;             // the step token whose input becomes state entry s
    fresh[s] = q >= 0 ? (q < m ? vals[K - 1 + q] : input(q)) : vals[s + count];
  }
  for (int s = 0; s < K - 1; ++s) st[(long long)s * a.channels] = fresh[s];
}

// The same for a number of taps known when the kernel is compiled (2 to 4): a thread walks CONV_RUN neighbouring tokens of
// one channel and keeps the inputs it has fetched as the next tokens' window, so an input is read about once instead of
// once per tap, and the taps' weights once per run.  A sequence's first step tokens (the ones whose taps reach before the
// step) are still all done by the thread that meets the sequence's first token, state first, new state last.
constexpr int CONV_RUN = 8;

template <typename O2, int K>
__global__ void __launch_bounds__(128) causal_conv_run_kernel(ConvArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_first = blockIdx.x * CONV_RUN;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const float ib = a.in_bias ? a.in_bias[c] : 0.f, ob = a.bias ? a.bias[c] : 0.f;
  float w[K];
#pragma unroll
  for (int j = 0; j < K; ++j) w[j] = a.weight[(long long)c * K + j];
  auto fetch = [&](int token) {                    // the input at packed token `token`
    const float* r = a.rows + (long long)token * a.row_width + a.col0 + c;
    float v = r[0];
    for (int s = 1; s < a.n_partials; ++s) v += r[s * a.partial_stride];
    return v + ib;
  };
  O2* out2 = (O2*)a.out2;
  float win[K - 1];                                // win[d - 1]: the input of the token d before the current one
  int have = 0;                                    // how many of them are held
  const int n_last = n_first + CONV_RUN < a.n_tokens ? n_first + CONV_RUN : a.n_tokens;
  for (int n = n_first; n < n_last; ++n) {
    const int b = a.seq_of_token[n];
    const int t0 = a.cu_tokens[b];
    const int p = n - t0;
    if (p < K - 1) {
      have = 0;                                    // the window does not reach across a sequence's start
      if (p > 0) continue;                         // done with the sequence's first step token
      const int count = a.cu_tokens[b + 1] - t0;
      float vals[2 * K];
      float* st = a.state + (long long)a.slots[b] * (K - 1) * a.channels + c;
      const int lb = a.len_before[b];
#pragma unroll
      for (int s = 0; s < K - 1; ++s) vals[s] = (lb - (K - 1) + s >= 0) ? st[(long long)s * a.channels] : 0.f;
      const int m = count < K - 1 ? count : K - 1;
#pragma unroll
      for (int q = 0; q < K - 1; ++q) vals[K - 1 + q] = q < m ? fetch(t0 + q) : 0.f;
#pragma unroll
      for (int q = 0; q < K - 1; ++q) {
        if (q < m) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < K; ++j) acc = fmaf(w[j], vals[q + j], acc);
          acc += ob;
          a.out[(long long)(t0 + q) * a.channels + c] = acc;
          if (out2) out2[(long long)(t0 + q) * a.channels + c] = from_f32<O2>(acc);
        }
      }
      float fresh[K - 1];
#pragma unroll
      for (int s = 0; s < K - 1; ++s) {
        const int q = count - (K - 1) + s;         // the step token whose input becomes state entry s
        float v;
        if (q >= m) v = fetch(t0 + q);
        else {
          v = 0.f;
#pragma unroll
          for (int e = 0; e < 2 * K - 2; ++e)      // vals[s + count] (q < 0) or vals[K - 1 + q], without a runtime index
            if (e == (q >= 0 ? K - 1 + q : s + count)) v = vals[e];
        }
        fresh[s] = v;
      }
#pragma unroll
      for (int s = 0; s < K - 1; ++s) st[(long long)s * a.channels] = fresh[s];
      continue;
    }
    const float x = fetch(n);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int d = K - 1 - j;                     // tap j weighs the token d before
      const float v = d <= have ? win[d - 1] : fetch(n - d);
      acc = fmaf(w[j], v, acc);
    }
    acc = fmaf(w[K - 1], x, acc) + ob;
    a.out[(long long)n * a.channels + c] = acc;
    if (out2) out2[(long long)n * a.channels + c] = from_f32<O2>(acc);
#pragma unroll
    for (int d = K - 2; d > 0; --d) win[d] = win[d - 1];
    win[0] = x;
    if (have < K - 1) ++have;
  }
}

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// MODE as in mingru_scan_kernel.
template <typename OT, int MODE>
__global__ void __launch_bounds__(128) rglru_scan_kernel(RgLruArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int piece = blockIdx.y, b = blockIdx.z;
  if (ch >= a.size) return;
  const int t_begin = a.cu_tokens[b], t_end = a.cu_tokens[b + 1];
  int lo = t_begin, hi = t_end;
  if (MODE != 0) {
    lo = t_begin + piece * LLG_MINGRU_PIECE;
    if (lo > t_end) lo = t_end;
    hi = (piece == a.pieces - 1 || lo + LLG_MINGRU_PIECE > t_end) ? t_end : lo + LLG_MINGRU_PIECE;
  }
  float* cr = MODE != 0 ? a.carry + (((long long)b * a.pieces + piece) * 2) * a.size + ch : nullptr;
  const int bw = a.block_width;
  const int blk = ch / bw, o = ch - blk * bw;
  const long long gcol = (long long)blk * 2 * bw + o;        // r's argument; i's lies bw further
  const float br = a.gate_bias[gcol], bi = a.gate_bias[gcol + bw];
  const float by = a.y_bias ? a.y_bias[ch] : 0.f;
  const float rate = -a.decay_scale * softplus_f(a.lam[ch]);
  float S = 0.f, A = 1.f;
  if (MODE == 0) S = a.state[(long long)a.slots[b] * a.size + ch];
  if (MODE == 2) {
    if (lo >= hi) return;
    S = cr[a.size];
  }
  OT* out = (OT*)a.out;
  const long long grow = 2LL * a.size;
  for (int n0 = lo; n0 < hi; n0 += SCAN_BATCH) {
    float gr[SCAN_BATCH], gi[SCAN_BATCH], u[SCAN_BATCH], y[SCAN_BATCH];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (n0 + k < hi) {
        gr[k] = a.gates[(n0 + k) * grow + gcol] + br;
        gi[k] = a.gates[(n0 + k) * grow + gcol + bw] + bi;
        u[k] = a.u[(long long)(n0 + k) * a.size + ch];
        y[k] = by;
      }
    }
    if (MODE != 1) {
      for (int s = 0; s < a.n_partials; ++s) {
        const float* p = a.rows + s * a.partial_stride + (long long)n0 * a.row_width + a.y_col + ch;
#pragma unroll
        for (int k = 0; k < SCAN_BATCH; ++k)
          if (n0 + k < hi) y[k] += p[(long long)k * a.row_width];
      }
    }
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (n0 + k < hi) {
        const float r = sigmoid_f(gr[k]), i = sigmoid_f(gi[k]);
        const float la = rate * r;
        const float at = expf(la);
        const float drive = sqrtf(-expm1f(2.0f * la)) * i * u[k];      // sqrt(1 - a^2) without the cancellation near a = 1
        S = at * S + drive;
        if (MODE == 1) A *= at;
        else out[(long long)(n0 + k) * a.size + ch] = from_f32<OT>(S * llg_act(1, y[k]));
      }
    }
  }
  if (MODE == 0) a.state[(long long)a.slots[b] * a.size + ch] = S;
  if (MODE == 1) {
    cr[0] = A;
    cr[a.size] = S;
  }
}

template <typename OT>
int rglru_launch(const RgLruArgs& a, cudaStream_t stream) {
  const unsigned cb = (unsigned)((a.size + 127) / 128);
  if (!a.carry) {
    llg_launch(rglru_scan_kernel<OT, 0>, dim3(cb, 1, a.n_seqs), dim3(128), 0, stream, a);
    return llg_check_launch("rglru_scan");
  }
  MinGruArgs j;
  memset(&j, 0, sizeof(j));
  j.state = a.state;
  j.slots = a.slots;
  j.carry = a.carry;
  j.pieces = a.pieces;
  j.size = a.size;
  llg_launch(rglru_scan_kernel<OT, 1>, dim3(cb, a.pieces, a.n_seqs), dim3(128), 0, stream, a);
  llg_launch(mingru_join_kernel, dim3(cb, a.n_seqs), dim3(128), 0, stream, j);
  llg_launch(rglru_scan_kernel<OT, 2>, dim3(cb, a.pieces, a.n_seqs), dim3(128), 0, stream, a);
  return llg_check_launch("rglru_scan (pieces)");
}

constexpr int RET_THREADS = 256;

// Shared memory: S [dim * vdim] | q [dim] | k [dim] | v [vdim] | g [vdim] | partial o [slices * vdim].
// MODE 0: the whole sequence from state[slot]; MODE 1: a piece from zero, its state to carry; MODE 2: a piece from carry.
template <typename OT, int MODE>
__global__ void __launch_bounds__(RET_THREADS) retention_kernel(RetentionArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  __shared__ float part[32];
  const int h = blockIdx.x, piece = blockIdx.y, b = blockIdx.z;
  const int dim = a.dim, vdim = a.vdim, nst = dim * vdim;
  const int slices = RET_THREADS / vdim > 0 ? RET_THREADS / vdim : 1;
  const int cols = RET_THREADS / slices;
  const int sl = threadIdx.x / cols, tj = threadIdx.x - sl * cols;
  float* S = smem;
  float* sq = S + nst;
  float* sk = sq + dim;
  float* sv = sk + dim;
  float* sg = sv + vdim;
  float* so = sg + vdim;
  const int t_begin = a.cu_tokens[b], t_end = a.cu_tokens[b + 1];
  int lo = t_begin, hi = t_end;
  if (MODE != 0) {
    lo = t_begin + piece * LLG_RETENTION_PIECE;
    if (lo > t_end) lo = t_end;
    hi = (piece == a.pieces - 1 || lo + LLG_RETENTION_PIECE > t_end) ? t_end : lo + LLG_RETENTION_PIECE;
  }
  float* gstate = a.state + ((long long)a.slots[b] * a.nh + h) * nst;
  float* cr = MODE != 0 ? a.carry + (((long long)b * a.pieces + piece) * a.nh + h) * nst : nullptr;
  if (MODE == 2 && lo >= hi) return;
  for (int e = threadIdx.x; e < nst; e += RET_THREADS) S[e] = MODE == 0 ? gstate[e] : MODE == 1 ? 0.f : cr[e];
  const float decay = a.decay[h];
  const int rd = a.cos_table ? a.rotary_dim : 0, half = rd / 2;
  OT* out = (OT*)a.out;
  for (int n = lo; n < hi; ++n) {
    const float* row = a.rows + (long long)n * a.row_width;
    auto summed = [&](int col) {
      float v = row[col];
      for (int s = 1; s < a.n_partials; ++s) v += row[s * a.partial_stride + col];
      return v;
    };
    int pos = a.positions[n];
    if (pos >= a.table_positions) pos = a.table_positions - 1;
    for (int i = threadIdx.x; i < dim; i += RET_THREADS) {
      float kv = summed(a.k_col + h * dim + i);
      float qv = MODE != 1 ? summed(a.q_col + h * dim + i) : 0.f;
      if (i < rd) {
        const int f = i < half ? i : i - half;
        const int ip = i < half ? i + half : i - half;
        const float c = a.cos_table[(long long)pos * half + f], s = a.sin_table[(long long)pos * half + f];
        const float kp = summed(a.k_col + h * dim + ip);
        kv = i < half ? kv * c - kp * s : kv * c + kp * s;
        if (MODE != 1) {
          const float qp = summed(a.q_col + h * dim + ip);
          qv = i < half ? qv * c - qp * s : qv * c + qp * s;
        }
      }
      sk[i] = kv * a.k_scale;
      sq[i] = qv;
    }
    for (int j = threadIdx.x; j < vdim; j += RET_THREADS) {
      sv[j] = summed(a.v_col + h * vdim + j);
      if (MODE != 1) sg[j] = summed(a.g_col + h * vdim + j);
    }
    __syncthreads();
    // threads beyond slices * cols (where the block's size is no multiple of cols) have no share of the state
    for (int j = sl < slices ? tj : vdim; j < vdim; j += cols) {
      const float vj = sv[j];
      float o = 0.f;
      for (int i = sl; i < dim; i += slices) {
        const float s = fmaf(decay, S[i * vdim + j], sk[i] * vj);
        S[i * vdim + j] = s;
        o = fmaf(s, sq[i], o);
      }
      if (MODE != 1) so[sl * vdim + j] = o;
    }
    if (MODE != 1) {
      __syncthreads();
      float ss = 0.f;
      for (int j = threadIdx.x; j < vdim; j += RET_THREADS) {
        float o = so[j];
        for (int s = 1; s < slices; ++s) o += so[s * vdim + j];
        so[j] = o;
        ss = fmaf(o, o, ss);
      }
      ss = block_sum(ss, part);
      const float inv = 1.0f / sqrtf(ss / (float)vdim + a.eps);
      for (int j = threadIdx.x; j < vdim; j += RET_THREADS) {
        const float g = sg[j];
        out[((long long)n * a.nh + h) * vdim + j] = from_f32<OT>(so[j] * inv * (g / (1.0f + expf(-g))));
      }
    }
    __syncthreads();
  }
  if (MODE == 0)
    for (int e = threadIdx.x; e < nst; e += RET_THREADS) gstate[e] = S[e];
  if (MODE == 1)
    for (int e = threadIdx.x; e < nst; e += RET_THREADS) cr[e] = S[e];
}

// The same walk with the state in registers and the tokens taken RET_BATCH at a time: the batch's q, k (rotated), v and
// gate arguments are summed into shared memory together, so that no token waits for memory on its own; a thread owns
// column j of R neighbouring rows of the state (rows sl * R ...; q and k rows in shared memory are filled with zeros up
// to slices * R elements, so the walk needs no bounds and reads four elements an access), and the walk through a batch
// needs no barrier; every token's partial read-outs (one per slice) are left in shared memory and the batch's unit
// norms and gates are done together, a warp per token.  For value heads of up to THREADS elements.
constexpr int RET_BATCH = 16;

template <typename OT, int MODE, int R, int THREADS>
__global__ void __launch_bounds__(THREADS) retention_reg_kernel(RetentionArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int h = blockIdx.x, piece = blockIdx.y, b = blockIdx.z;
  const int dim = a.dim, vdim = a.vdim, nst = dim * vdim;
  const int slices = THREADS / vdim;
  const int dp = slices * R;                 // padded length of a q or k row (a multiple of four, at least dim)
  const bool active = threadIdx.x < slices * vdim;
  const int sl = threadIdx.x / vdim, j = threadIdx.x - sl * vdim;
  float* sq = smem;                          // [RET_BATCH][dp]
  float* sk = sq + RET_BATCH * dp;           // [RET_BATCH][dp]
  float* sv = sk + RET_BATCH * dp;           // [RET_BATCH][vdim]
  float* sg = sv + RET_BATCH * vdim;         // [RET_BATCH][vdim]
  float* po = sg + RET_BATCH * vdim;         // [RET_BATCH][slices][vdim]
  const int t_begin = a.cu_tokens[b], t_end = a.cu_tokens[b + 1];
  int lo = t_begin, hi = t_end;
  if (MODE != 0) {
    lo = t_begin + piece * LLG_RETENTION_PIECE;
    if (lo > t_end) lo = t_end;
    hi = (piece == a.pieces - 1 || lo + LLG_RETENTION_PIECE > t_end) ? t_end : lo + LLG_RETENTION_PIECE;
  }
  float* gstate = a.state + ((long long)a.slots[b] * a.nh + h) * nst;
  float* cr = MODE != 0 ? a.carry + (((long long)b * a.pieces + piece) * a.nh + h) * nst : nullptr;
  if (MODE == 2 && lo >= hi) return;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = sl * R + r;
    S[r] = (active && i < dim && MODE != 1) ? (MODE == 0 ? gstate : cr)[i * vdim + j] : 0.f;
  }
  const float decay = a.decay[h];
  const int rd = a.cos_table ? a.rotary_dim : 0, half = rd / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  OT* out = (OT*)a.out;
  for (int n0 = lo; n0 < hi; n0 += RET_BATCH) {
    const int nb = hi - n0 < RET_BATCH ? hi - n0 : RET_BATCH;
    for (int idx = threadIdx.x; idx < nb * dp; idx += THREADS) {
      const int t = idx / dp, i = idx - t * dp;
      float kv = 0.f, qv = 0.f;
      if (i < dim) {
        const float* row = a.rows + (long long)(n0 + t) * a.row_width;
        auto summed = [&](int col) {
          float v = row[col];
          for (int s = 1; s < a.n_partials; ++s) v += row[s * a.partial_stride + col];
          return v;
        };
        kv = summed(a.k_col + h * dim + i);
        if (MODE != 1) qv = summed(a.q_col + h * dim + i);
        if (i < rd) {
          int pos = a.positions[n0 + t];
          if (pos >= a.table_positions) pos = a.table_positions - 1;
          const int f = i < half ? i : i - half;
          const int ip = i < half ? i + half : i - half;
          const float c = a.cos_table[(long long)pos * half + f], sn = a.sin_table[(long long)pos * half + f];
          const float kp = summed(a.k_col + h * dim + ip);
          kv = i < half ? kv * c - kp * sn : kv * c + kp * sn;
          if (MODE != 1) {
            const float qp = summed(a.q_col + h * dim + ip);
            qv = i < half ? qv * c - qp * sn : qv * c + qp * sn;
          }
        }
      }
      sk[idx] = kv * a.k_scale;
      sq[idx] = qv;
    }
    for (int idx = threadIdx.x; idx < nb * vdim; idx += THREADS) {
      const int t = idx / vdim, c = idx - t * vdim;
      const float* row = a.rows + (long long)(n0 + t) * a.row_width;
      float v = row[a.v_col + h * vdim + c];
      for (int s = 1; s < a.n_partials; ++s) v += row[s * a.partial_stride + a.v_col + h * vdim + c];
      sv[idx] = v;
      if (MODE != 1) {
        float g = row[a.g_col + h * vdim + c];
        for (int s = 1; s < a.n_partials; ++s) g += row[s * a.partial_stride + a.g_col + h * vdim + c];
        sg[idx] = g;
      }
    }
    __syncthreads();
    if (active) {
      for (int t = 0; t < nb; ++t) {
        const float vj = sv[t * vdim + j];
        const float4* kt = reinterpret_cast<const float4*>(sk + t * dp + sl * R);
        const float4* qt = reinterpret_cast<const float4*>(sq + t * dp + sl * R);
        float o = 0.f;
#pragma unroll
        for (int r4 = 0; r4 < R / 4; ++r4) {
          const float4 kk = kt[r4];
          float sn;
          if (MODE != 1) {
            const float4 qq = qt[r4];
            sn = fmaf(decay, S[4 * r4], kk.x * vj); S[4 * r4] = sn; o = fmaf(sn, qq.x, o);
            sn = fmaf(decay, S[4 * r4 + 1], kk.y * vj); S[4 * r4 + 1] = sn; o = fmaf(sn, qq.y, o);
            sn = fmaf(decay, S[4 * r4 + 2], kk.z * vj); S[4 * r4 + 2] = sn; o = fmaf(sn, qq.z, o);
            sn = fmaf(decay, S[4 * r4 + 3], kk.w * vj); S[4 * r4 + 3] = sn; o = fmaf(sn, qq.w, o);
          } else {
            S[4 * r4] = fmaf(decay, S[4 * r4], kk.x * vj);
            S[4 * r4 + 1] = fmaf(decay, S[4 * r4 + 1], kk.y * vj);
            S[4 * r4 + 2] = fmaf(decay, S[4 * r4 + 2], kk.z * vj);
            S[4 * r4 + 3] = fmaf(decay, S[4 * r4 + 3], kk.w * vj);
          }
        }
        if (MODE != 1) po[(t * slices + sl) * vdim + j] = o;
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int t = warp; t < nb; t += THREADS / 32) {
        float ss = 0.f;
        for (int c = lane; c < vdim; c += 32) {
          float o = po[t * slices * vdim + c];
          for (int s = 1; s < slices; ++s) o += po[(t * slices + s) * vdim + c];
          po[t * slices * vdim + c] = o;
          ss = fmaf(o, o, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + a.eps);
        for (int c = lane; c < vdim; c += 32) {
          const float g = sg[t * vdim + c];
          out[((long long)(n0 + t) * a.nh + h) * vdim + c] = from_f32<OT>(po[t * slices * vdim + c] * inv * (g / (1.0f + expf(-g))));
        }
      }
    }
    __syncthreads();
  }
  if (MODE != 2 && active) {
    float* dst = MODE == 0 ? gstate : cr;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = sl * R + r;
      if (i < dim) dst[i * vdim + j] = S[r];
    }
  }
}

// Walks a sequence's pieces: piece p starts from what the pieces before it make of the sequence's state.  The states the
// pieces reached are fetched SCAN_BATCH at a time, ahead of the chain of multiplications.
__global__ void __launch_bounds__(256) retention_join_kernel(RetentionArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, b = blockIdx.z;
  const int nst = a.dim * a.vdim;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nst) return;
  const float decay = a.decay[h];
  const int t_begin = a.cu_tokens[b], t_end = a.cu_tokens[b + 1];
  float* st = a.state + ((long long)a.slots[b] * a.nh + h) * nst + e;
  float S = *st;
  // decay^LLG_RETENTION_PIECE by the same chain of roundings as a walk through a whole piece
  float whole = 1.f;
  for (int t = 0; t < LLG_RETENTION_PIECE; ++t) whole *= decay;
  const long long step = (long long)a.nh * nst;
  float* cr = a.carry + (((long long)b * a.pieces) * a.nh + h) * nst + e;
  for (int p0 = 0; p0 < a.pieces; p0 += SCAN_BATCH, cr += SCAN_BATCH * step) {
    float reached[SCAN_BATCH];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k)
      if (p0 + k < a.pieces) reached[k] = cr[k * step];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      const int p = p0 + k;
      if (p < a.pieces) {
        int lo = t_begin + p * LLG_RETENTION_PIECE;
        if (lo > t_end) lo = t_end;
        const int hi = (p == a.pieces - 1 || lo + LLG_RETENTION_PIECE > t_end) ? t_end : lo + LLG_RETENTION_PIECE;
        float A = whole;
        if (hi - lo != LLG_RETENTION_PIECE) {
          A = 1.f;
          for (int t = lo; t < hi; ++t) A *= decay;
        }
        cr[k * step] = S;
        S = A * S + reached[k];
      }
    }
  }
  *st = S;
}

template <typename K>
int retention_attr(K kernel, size_t smem) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llg_fail("retention: shared memory %zu: %s", smem, cudaGetErrorString(e));
  }
  return 0;
}

// KERNEL(MODE): the kernel of a mode, whichever form.
#define RET_RUN(KERNEL, SMEM, THREADS)                                                                                 \
  do {                                                                                                          \
    if (!a.carry) {                                                                                             \
      if (retention_attr(KERNEL(0), SMEM)) return 1;                                                            \
      llg_launch(KERNEL(0), dim3(a.nh, 1, a.n_seqs), dim3(THREADS), SMEM, stream, a);                           \
      return llg_check_launch("retention");                                                                     \
    }                                                                                                           \
    if (retention_attr(KERNEL(1), SMEM) || retention_attr(KERNEL(2), SMEM)) return 1;                           \
    llg_launch(KERNEL(1), dim3(a.nh, a.pieces, a.n_seqs), dim3(THREADS), SMEM, stream, a);                      \
    llg_launch(retention_join_kernel, dim3((nst + 255) / 256, a.nh, a.n_seqs), dim3(256), 0, stream, a);        \
    llg_launch(KERNEL(2), dim3(a.nh, a.pieces, a.n_seqs), dim3(THREADS), SMEM, stream, a);                      \
    return llg_check_launch("retention (pieces)");                                                              \
  } while (0)

template <typename OT>
int retention_launch(const RetentionArgs& a, size_t smem, cudaStream_t stream) {
  const int nst = a.dim * a.vdim;
  // The state in registers where a thread's share of it is at most 32 rows of one column: with 256 threads, or with
  // 512 where that halves a share of more than 32 rows.
  for (int threads = RET_THREADS; threads <= 2 * RET_THREADS; threads *= 2) {
    if (a.vdim > threads) continue;
    const int slices = threads / a.vdim;
    const int rows = (a.dim + slices - 1) / slices;
    if (rows > 32) continue;
    const int r = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    const size_t reg_smem = (size_t)RET_BATCH * (2 * slices * r + 2 * a.vdim + slices * a.vdim) * sizeof(float);
    if (reg_smem > 200 * 1024) continue;
#define K4(M) retention_reg_kernel<OT, M, 4, 256>
#define K8(M) retention_reg_kernel<OT, M, 8, 256>
#define K16(M) retention_reg_kernel<OT, M, 16, 256>
#define K32(M) retention_reg_kernel<OT, M, 32, 256>
#define K4W(M) retention_reg_kernel<OT, M, 4, 512>
#define K8W(M) retention_reg_kernel<OT, M, 8, 512>
#define K16W(M) retention_reg_kernel<OT, M, 16, 512>
#define K32W(M) retention_reg_kernel<OT, M, 32, 512>
    if (threads == RET_THREADS) {
      if (r == 4) RET_RUN(K4, reg_smem, 256);
      else if (r == 8) RET_RUN(K8, reg_smem, 256);
      else if (r == 16) RET_RUN(K16, reg_smem, 256);
      else RET_RUN(K32, reg_smem, 256);
    } else {
      if (r == 4) RET_RUN(K4W, reg_smem, 512);
      else if (r == 8) RET_RUN(K8W, reg_smem, 512);
      else if (r == 16) RET_RUN(K16W, reg_smem, 512);
      else RET_RUN(K32W, reg_smem, 512);
    }
#undef K4
#undef K8
#undef K16
#undef K32
#undef K4W
#undef K8W
#undef K16W
#undef K32W
  }
#define KS(M) retention_kernel<OT, M>
  RET_RUN(KS, smem, RET_THREADS);
#undef KS
}
#undef RET_RUN

}  // namespace

LLG_API int llg_conv_max_taps() { return LLG_CONV_MAX_TAPS; }
LLG_API int llg_retention_piece() { return LLG_RETENTION_PIECE; }

LLG_API int llg_causal_conv(const ConvArgs* args, cudaStream_t stream) {
  const ConvArgs& a = *args;
  LLG_REQUIRE(a.n_seqs >= 0 && a.n_tokens >= 0 && a.channels > 0 && a.n_partials >= 1, "causal_conv: bad sizes");
  LLG_REQUIRE(a.taps >= 1 && a.taps <= LLG_CONV_MAX_TAPS, "causal_conv: %d taps (1 to %d)", a.taps, LLG_CONV_MAX_TAPS);
  LLG_REQUIRE(a.col0 >= 0 && a.col0 + a.channels <= a.row_width, "causal_conv: %d channels at column %d of %d", a.channels, a.col0, a.row_width);
  LLG_REQUIRE(a.taps == 1 || a.state, "causal_conv: more than one tap needs the sequences' state");
  if (a.n_tokens == 0) return 0;
  dim3 grid(a.n_tokens, (a.channels + 127) / 128);
  LLG_REQUIRE(grid.y <= 65535, "causal_conv: too many channels");
  LLG_REQUIRE(!a.out2 || a.out2_dtype == LLG_F32 || a.out2_dtype == LLG_BF16, "causal_conv: unknown output type %d", a.out2_dtype);
  const bool bf = a.out2 && a.out2_dtype == LLG_BF16;
  // steps of many tokens and 2 to 4 taps: runs of tokens a thread
  if (a.taps >= 2 && a.taps <= 4 && a.n_tokens >= 4 * CONV_RUN) {
    dim3 runs((a.n_tokens + CONV_RUN - 1) / CONV_RUN, grid.y);
#define CONV_RUN_LAUNCH(K)                                                                               \
  do {                                                                                                   \
    if (bf) llg_launch(causal_conv_run_kernel<__nv_bfloat16, K>, runs, dim3(128), 0, stream, a);         \
    else llg_launch(causal_conv_run_kernel<float, K>, runs, dim3(128), 0, stream, a);                    \
  } while (0)
    if (a.taps == 2) CONV_RUN_LAUNCH(2);
    else if (a.taps == 3) CONV_RUN_LAUNCH(3);
    else CONV_RUN_LAUNCH(4);
#undef CONV_RUN_LAUNCH
    return llg_check_launch("causal_conv (runs)");
  }
  if (bf) llg_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, a);
  else llg_launch(causal_conv_kernel<float>, grid, dim3(128), 0, stream, a);
  return llg_check_launch("causal_conv");
}

LLG_API int llg_rglru_scan(const RgLruArgs* args, int max_count, cudaStream_t stream) {
  const RgLruArgs& a = *args;
  LLG_REQUIRE(a.n_seqs >= 0 && a.n_tokens >= 0 && a.size > 0 && a.n_partials >= 1, "rglru_scan: bad sizes");
  LLG_REQUIRE(a.block_width > 0 && a.size % a.block_width == 0, "rglru_scan: %d channels in blocks of %d", a.size, a.block_width);
  LLG_REQUIRE(a.y_col >= 0 && a.y_col + a.size <= a.row_width, "rglru_scan: %d channels at column %d of %d", a.size, a.y_col, a.row_width);
  LLG_REQUIRE(a.n_seqs <= 65535, "rglru_scan: %d sequences in a step (at most 65535)", a.n_seqs);
  if (a.carry)
    LLG_REQUIRE(a.pieces >= 1 && a.pieces <= 65535 && (long long)a.pieces * LLG_MINGRU_PIECE >= max_count,
                "rglru_scan: %d pieces of %d tokens do not hold a sequence of %d", a.pieces, LLG_MINGRU_PIECE, max_count);
  if (a.n_seqs == 0 || a.n_tokens == 0) return 0;
  if (a.out_dtype == LLG_F32) return rglru_launch<float>(a, stream);
  if (a.out_dtype == LLG_BF16) return rglru_launch<__nv_bfloat16>(a, stream);
  return llg_fail("rglru_scan: unknown output type %d", a.out_dtype);
}

LLG_API int llg_retention(const RetentionArgs* args, int max_count, cudaStream_t stream) {
  const RetentionArgs& a = *args;
  LLG_REQUIRE(a.n_seqs >= 0 && a.n_tokens >= 0 && a.nh > 0 && a.dim > 0 && a.vdim > 0 && a.n_partials >= 1, "retention: bad sizes");
  LLG_REQUIRE(a.n_seqs <= 65535 && a.nh <= 65535, "retention: too many sequences or heads");
  LLG_REQUIRE(!a.cos_table || (a.rotary_dim > 0 && a.rotary_dim % 2 == 0 && a.rotary_dim <= a.dim && a.table_positions > 0),
              "retention: %d rotated elements of a head of %d", a.rotary_dim, a.dim);
  LLG_REQUIRE(a.eps > 0.f, "retention: eps %g", a.eps);
  if (a.carry)
    LLG_REQUIRE(a.pieces >= 1 && a.pieces <= 65535 && (long long)a.pieces * LLG_RETENTION_PIECE >= max_count,
                "retention: %d pieces of %d tokens do not hold a sequence of %d", a.pieces, LLG_RETENTION_PIECE, max_count);
  const int slices = RET_THREADS / a.vdim > 0 ? RET_THREADS / a.vdim : 1;
  const size_t smem = ((size_t)a.dim * a.vdim + 2 * (size_t)a.dim + 2 * (size_t)a.vdim + (size_t)slices * a.vdim) * sizeof(float);
  LLG_REQUIRE(smem <= 220 * 1024, "retention: a head's state of %d x %d does not fit shared memory", a.dim, a.vdim);
  if (a.n_seqs == 0 || a.n_tokens == 0) return 0;
  if (a.out_dtype == LLG_F32) return retention_launch<float>(a, smem, stream);
  if (a.out_dtype == LLG_BF16) return retention_launch<__nv_bfloat16>(a, smem, stream);
  return llg_fail("retention: unknown output type %d", a.out_dtype);
}
