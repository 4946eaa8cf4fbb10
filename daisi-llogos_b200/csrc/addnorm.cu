// Norms around a residual that takes several terms at once, and the embedding and per-token input that go with them
// (argument blocks in kernel_args.h).
//
//   multi_add_rmsnorm : residual += sum over terms of scale_t * [RMS norm with a weight of] (sum of the term's partials);
//                       then up to two outputs of the same row: normed with a weight each (plus an offset: a weight kept
//                       as its difference from one), or the row as it is in the output type.  One block per row; the row lies in shared
//                       memory as float32 between the passes.
//   hash_embed        : scale * table[token] + pair_table[hash(previous token, token)], RMS-normed into the residual; the
//                       previous token of a step's first token comes from, and the step's last token goes to, a per-slot
//                       state.
//   table_gate        : act(partials) * a slice of a per-token table row.
//
// Every sum, statistic and the residual are float32.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }
LLG_API int llg_addnorm_max_terms() { return LLG_ADDNORM_TERMS; }
LLG_API int llg_addnorm_max_outs() { return LLG_ADDNORM_OUTS; }

namespace {

template <int VEC> struct Pack { float v[VEC]; };

template <int VEC> __device__ __forceinline__ Pack<VEC> load_f32(const float* p) {
  Pack<VEC> r;
  if (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[VEC > 1 ? 1 : 0] = t.y; r.v[VEC > 2 ? 2 : 0] = t.z; r.v[VEC > 3 ? 3 : 0] = t.w; }
  else r.v[0] = *p;
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

// VEC 4: every access moves four neighbouring elements (the host has checked sizes and addresses).  A term's partial sums
// are fetched four sets at a time, so that the few rows of a decode step do not wait for one load after another.
template <typename OT, int VEC>
__global__ void __launch_bounds__(1024) multi_add_rmsnorm_kernel(AddNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  __shared__ float part[32];
  const int hidden = a.hidden;
  float* row = smem;
  float* tmp = smem + hidden;
  const int j = blockIdx.x;
  const int r = a.rows ? a.rows[j] : j;
  float* res = a.residual + (long long)r * hidden;
  const int first = threadIdx.x * VEC, stride = blockDim.x * VEC;
  // every thread owns the same elements of the row in every pass, so the passes need no barrier of their own
  for (int i = first; i < hidden; i += stride) store<VEC>(row + i, load_f32<VEC>(res + i));
  for (int t = 0; t < a.n_terms; ++t) {
    const AddNormTerm& term = a.terms[t];
    const float* p = term.data + (long long)r * hidden;
    float ss = 0.f;
    for (int i = first; i < hidden; i += stride) {
      Pack<VEC> y = load_f32<VEC>(p + i);
      int s = 1;
      for (; s + 3 < term.n_partials; s += 4) {
        const Pack<VEC> y0 = load_f32<VEC>(p + s * a.partial_stride + i), y1 = load_f32<VEC>(p + (s + 1) * a.partial_stride + i);
        const Pack<VEC> y2 = load_f32<VEC>(p + (s + 2) * a.partial_stride + i), y3 = load_f32<VEC>(p + (s + 3) * a.partial_stride + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) y.v[c] = (((y.v[c] + y0.v[c]) + y1.v[c]) + y2.v[c]) + y3.v[c];
      }
      for (; s < term.n_partials; ++s) {
        const Pack<VEC> y0 = load_f32<VEC>(p + s * a.partial_stride + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) y.v[c] += y0.v[c];
      }
      if (term.norm_w) {
        store<VEC>(tmp + i, y);
#pragma unroll
        for (int c = 0; c < VEC; ++c) ss = fmaf(y.v[c], y.v[c], ss);
      } else {
        Pack<VEC> v = load_f32<VEC>(row + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) v.v[c] += term.scale * y.v[c];
        store<VEC>(row + i, v);
      }
    }
    if (term.norm_w) {
      ss = block_sum(ss, part);
      const float inv = 1.0f / sqrtf(ss / (float)hidden + term.norm_eps);
      for (int i = first; i < hidden; i += stride) {
        Pack<VEC> v = load_f32<VEC>(row + i);
        const Pack<VEC> y = load_f32<VEC>(tmp + i), w = load_f32<VEC>(term.norm_w + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) v.v[c] += term.scale * (y.v[c] * inv * w.v[c]);
        store<VEC>(row + i, v);
      }
    }
  }
  float ss = 0.f;
  for (int i = first; i < hidden; i += stride) {
    const Pack<VEC> v = load_f32<VEC>(row + i);
    if (a.n_terms) store<VEC>(res + i, v);
#pragma unroll
    for (int c = 0; c < VEC; ++c) ss = fmaf(v.v[c], v.v[c], ss);
  }
  bool normed = false;
  for (int o = 0; o < a.n_outs; ++o) normed = normed || a.outs[o].weight != nullptr;
  float inv = 1.f;
  if (normed) {
    ss = block_sum(ss, part);
    inv = 1.0f / sqrtf(ss / (float)hidden + a.eps);
  }
  for (int o = 0; o < a.n_outs; ++o) {
    OT* out = (OT*)a.outs[o].out + (long long)j * hidden;
    const float* w = a.outs[o].weight;
    const float off = a.outs[o].offset;
    for (int i = first; i < hidden; i += stride) {
      Pack<VEC> v = load_f32<VEC>(row + i);
      if (w) {
        const Pack<VEC> ww = load_f32<VEC>(w + i);
#pragma unroll
        for (int c = 0; c < VEC; ++c) v.v[c] = v.v[c] * inv * (off + ww.v[c]);
      }
      store<VEC>(out + i, v);
    }
  }
}

template <typename TT, typename PT>
__global__ void __launch_bounds__(1024) hash_embed_kernel(HashEmbedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float row[];
  __shared__ float part[32];
  __shared__ int pair_row;
  const int n = blockIdx.x;
  const int hidden = a.hidden;
  int tok = a.token_ids[n];
  if (tok < 0 || tok >= a.vocab) tok = 0;
  if (threadIdx.x == 0) {
    int pr = -1;
    if (a.pair_table) {
      const int b = a.seq_of_token[n];
      const int first = a.cu_tokens[b];
      int prev = 0;
      bool has_prev = a.positions[n] > 0;
      if (n > first) prev = a.token_ids[n - 1];
      else {
        // the sequence's first token of this step: the token before it is the state's, and the state moves on to the
        // step's last token (no other thread reads or writes this slot's entry)
        int* st = a.last_token + a.slots[b];
        if (has_prev) prev = *st;
        int last = a.token_ids[a.cu_tokens[b + 1] - 1];
        if (last < 0 || last >= a.vocab) last = 0;
        *st = last;
      }
      if (prev < 0 || prev >= a.vocab) prev = 0;
      if (!has_prev) pr = a.buckets;
      else pr = (int)((((long long)prev * (a.mul_prev % a.buckets)) % a.buckets + ((long long)tok * (a.mul_cur % a.buckets)) % a.buckets) % a.buckets);
      if (pr < 0) pr += a.buckets;
    }
    pair_row = pr;
  }
  __syncthreads();
  const TT* e = (const TT*)a.table + (long long)tok * hidden;
  const PT* pe = pair_row >= 0 ? (const PT*)a.pair_table + (long long)pair_row * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32(e[i]) * a.scale;
    if (pe) v += to_f32(pe[i]);
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  float* out = a.out + (long long)n * hidden;
  if (a.norm_w) {
    ss = block_sum(ss, part);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + a.eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = row[i] * inv * (a.norm_offset + a.norm_w[i]);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = row[i];
  }
}

template <typename TT, typename OT>
__global__ void __launch_bounds__(256) table_gate_kernel(TableGateArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)a.n_tokens * a.width) return;
  const int n = (int)(idx / a.width), j = (int)(idx % a.width);
  float z = 0.f;
  for (int s = 0; s < a.n_partials; ++s) z += a.rows[s * a.partial_stride + idx];
  int tok = a.token_ids[n];
  if (tok < 0 || tok >= a.vocab) tok = 0;
  const float e = to_f32(((const TT*)a.table)[(long long)tok * a.table_width + a.col0 + j]);
  ((OT*)a.out)[idx] = from_f32<OT>(llg_act(a.act, z) * e);
}

int threads_for(int hidden) {
  int t = (hidden + 3) / 4;
  t = (t + 31) / 32 * 32;
  return t < 128 ? 128 : (t > 1024 ? 1024 : t);
}

}  // namespace

LLG_API int llg_multi_add_rmsnorm(const AddNormArgs* args, cudaStream_t stream) {
  const AddNormArgs& a = *args;
  LLG_REQUIRE(a.n_out >= 0 && a.hidden > 0 && a.eps > 0.f, "multi_add_rmsnorm: bad sizes n_out=%d hidden=%d eps=%g", a.n_out, a.hidden, a.eps);
  LLG_REQUIRE(a.n_terms >= 0 && a.n_terms <= LLG_ADDNORM_TERMS, "multi_add_rmsnorm: %d terms (at most %d)", a.n_terms, LLG_ADDNORM_TERMS);
  LLG_REQUIRE(a.n_outs >= 1 && a.n_outs <= LLG_ADDNORM_OUTS, "multi_add_rmsnorm: %d outputs (1 to %d)", a.n_outs, LLG_ADDNORM_OUTS);
  for (int t = 0; t < a.n_terms; ++t) {
    LLG_REQUIRE(a.terms[t].data && a.terms[t].n_partials >= 1, "multi_add_rmsnorm: term %d has no partials", t);
    LLG_REQUIRE(!a.terms[t].norm_w || a.terms[t].norm_eps > 0.f, "multi_add_rmsnorm: term %d is normed with eps %g", t, a.terms[t].norm_eps);
  }
  if (a.n_out == 0) return 0;
  const size_t smem = 2 * (size_t)a.hidden * sizeof(float);
  LLG_REQUIRE(smem <= 200 * 1024, "multi_add_rmsnorm: rows of %d elements do not fit shared memory", a.hidden);
  auto aligned = [](const void* p) { return ((size_t)p % 16) == 0; };
  bool vec = a.hidden % 4 == 0 && a.partial_stride % 4 == 0 && aligned(a.residual);
  for (int t = 0; t < a.n_terms; ++t) vec = vec && aligned(a.terms[t].data) && aligned(a.terms[t].norm_w);
  for (int o = 0; o < a.n_outs; ++o) vec = vec && aligned(a.outs[o].out) && aligned(a.outs[o].weight);
  int threads = vec ? threads_for(a.hidden) : threads_for(4 * a.hidden);
  // many rows: smaller blocks, so that a multiprocessor holds several rows at different stages
  if (a.n_out > 2 * llg_sm_count() && threads > 256) threads = 256;
#define LAUNCH_V(OT, V)                                                                                           \
  do {                                                                                                            \
    auto k = multi_add_rmsnorm_kernel<OT, V>;                                                                     \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return llg_fail("multi_add_rmsnorm: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                             \
    llg_launch(k, dim3(a.n_out), dim3(threads), smem, stream, a);                                                 \
  } while (0)
#define LAUNCH(OT)            \
  do {                        \
    if (vec) LAUNCH_V(OT, 4); \
    else LAUNCH_V(OT, 1);     \
  } while (0)
  if (a.out_dtype == LLG_F32) LAUNCH(float);
  else if (a.out_dtype == LLG_BF16) LAUNCH(__nv_bfloat16);
  else return llg_fail("multi_add_rmsnorm: unknown output type %d", a.out_dtype);
#undef LAUNCH
#undef LAUNCH_V
  return llg_check_launch("multi_add_rmsnorm");
}

LLG_API int llg_hash_embed(const HashEmbedArgs* args, cudaStream_t stream) {
  const HashEmbedArgs& a = *args;
  LLG_REQUIRE(a.n_tokens >= 0 && a.hidden > 0 && a.vocab > 0, "hash_embed: bad sizes");
  LLG_REQUIRE(!a.pair_table || (a.buckets > 0 && a.last_token && a.seq_of_token && a.cu_tokens && a.slots && a.positions),
              "hash_embed: a pair table needs its buckets, the step's layout and the slots' last tokens");
  LLG_REQUIRE(!a.norm_w || a.eps > 0.f, "hash_embed: eps %g", a.eps);
  if (a.n_tokens == 0) return 0;
  const size_t smem = (size_t)a.hidden * sizeof(float);
  LLG_REQUIRE(smem <= 200 * 1024, "hash_embed: rows of %d elements do not fit shared memory", a.hidden);
  const int threads = threads_for(a.hidden);
  const int pd = a.pair_table ? a.pair_dtype : a.table_dtype;
#define LAUNCH(TT, PT)                                                                                       \
  do {                                                                                                       \
    auto k = hash_embed_kernel<TT, PT>;                                                                      \
    if (smem > 48 * 1024) {                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      if (e != cudaSuccess) return llg_fail("hash_embed: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                        \
    llg_launch(k, dim3(a.n_tokens), dim3(threads), smem, stream, a);                                         \
  } while (0)
  if (a.table_dtype == LLG_F32 && pd == LLG_F32) LAUNCH(float, float);
  else if (a.table_dtype == LLG_BF16 && pd == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (a.table_dtype == LLG_F32 && pd == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (a.table_dtype == LLG_BF16 && pd == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else return llg_fail("hash_embed: unknown table types %d, %d", a.table_dtype, pd);
#undef LAUNCH
  return llg_check_launch("hash_embed");
}

LLG_API int llg_table_gate(const TableGateArgs* args, cudaStream_t stream) {
  const TableGateArgs& a = *args;
  LLG_REQUIRE(a.n_tokens >= 0 && a.width > 0 && a.n_partials >= 1 && a.col0 >= 0 && a.col0 + a.width <= a.table_width && a.vocab > 0,
              "table_gate: bad sizes (width %d at column %d of %d)", a.width, a.col0, a.table_width);
  LLG_REQUIRE(a.act >= 0 && a.act < LLG_ACT_KINDS, "table_gate: unknown activation %d", a.act);
  if (a.n_tokens == 0) return 0;
  const unsigned grid = (unsigned)(((long long)a.n_tokens * a.width + 255) / 256);
#define LAUNCH(TT, OT) llg_launch(table_gate_kernel<TT, OT>, dim3(grid), dim3(256), 0, stream, a)
  if (a.table_dtype == LLG_F32 && a.out_dtype == LLG_F32) LAUNCH(float, float);
  else if (a.table_dtype == LLG_BF16 && a.out_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (a.table_dtype == LLG_F32 && a.out_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (a.table_dtype == LLG_BF16 && a.out_dtype == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else return llg_fail("table_gate: unknown types %d, %d", a.table_dtype, a.out_dtype);
#undef LAUNCH
  return llg_check_launch("table_gate");
}
