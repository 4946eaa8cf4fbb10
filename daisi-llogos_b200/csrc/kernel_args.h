// Argument blocks of the kernels' entry points that take more than a handful of values: plain structs that a caller
// fills and passes by address (Python through ctypes, the block runner in C++).  Every field is a device pointer, an
// int or a float; the layouts are part of the libraries' interface.
#pragma once

// What a norm leaves to the consumer of its output when it does not divide by the root mean square itself: the norm
// wrote x * weight and, per row, the sum of the row's squares, whole (parts = 1) or as `parts` partial sums (one per
// block of columns of whoever produced the row).  The consumer multiplies the rows of its product by
// 1 / sqrt(sum / width + eps): a product is linear in its rows, so the result is that of the normalised input, and
// nobody had to wait for a whole row before the product's operand could be written.
struct RowScale {
  const float* ss;            // [rows][parts], or null: rows are used as they are
  int parts;
  float inv_width;            // 1 / (elements of a row)
  float eps;
};

#ifdef __CUDACC__
// The first position that a query at position `pos` sees under a mask of size `window` (0: every position): its own
// chunk's first position, or the first of the last `window` positions.
__device__ __forceinline__ int mask_first(int pos, int window, int chunked) {
  if (window <= 0) return 0;
  return chunked ? (pos / window) * window : max(0, pos - window + 1);
}

__device__ __forceinline__ float row_scale_of(const RowScale& s, long long row) {
  if (!s.ss) return 1.0f;
  const float* p = s.ss + row * s.parts;
  float t = 0.f;
  for (int j0 = 0; j0 < s.parts; j0 += 8) {           // eight loads under way at a time; added in their order, so
    float v[8];                                       // the scale is the same whoever computes it
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = j0 + j < s.parts ? p[j0 + j] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += v[j];
  }
  return 1.0f / sqrtf(t * s.inv_width + s.eps);
}
#endif

struct QkPrepArgs {
  const void* qkv;            // [n_partials][n_tokens][(nh + 2 nkv) * hd], float32 or bfloat16
  int qkv_dtype;
  int n_partials;
  long long partial_stride;   // elements between partials
  const void* q_norm_w;       // [hd] or null
  const void* k_norm_w;       // [hd] or null
  int norm_w_dtype;
  float norm_eps;
  const void* bias;           // [(nh + 2 nkv) * hd] or null
  int bias_dtype;
  const float* cos_table;     // [positions][rotary_dim / 2] or null
  const float* sin_table;
  int rotary_dim;
  int pairing;                // 0: (i, i + rotary_dim/2), 1: (2i, 2i+1)
  int table_positions;
  const int* positions;       // [n_tokens]
  void* q_out;                // [n_tokens][nh][hd]
  void* k_new;                // [n_tokens][nkv][hd] or null
  void* v_new;
  void* k_pages;              // paged store or null
  void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* seq_of_token;    // [n_tokens] -> index into slots
  const int* slots;
  int n_tokens, nh, nkv, hd;
  RowScale row_scale;         // of the token rows of qkv (applied to the summed partials, before anything else)
  // Further forms; all zero gives the plain one.  Only the general kernel of elementwise.cu reads these (a caller
  // leaves them zero for the product whose epilogue is the preparation).
  int vd;                     // elements of a value head; 0 = hd.  A row of qkv then is nh*hd + nkv*hd + nkv*vd wide,
                              // and v_new / v_pages hold vd per head
  const float* v_mix;         // one number lam, or null: with v_first_in the values become (1 - lam) v + lam v_first_in
  const float* v_first_in;    // [n_tokens][nkv][vd] float32 or null
  float* v_first_out;         // [n_tokens][nkv][vd] float32 or null: receives the values as projected (before any blend)
};

// Attention for a step with several tokens per sequence (attention_simt.cu, attention_mma.cu, attention_tc.cu).
struct PrefillArgs {
  const void* q;            // [n_tokens][nh][hd]
  const void* k_new;        // [n_tokens][nkv][hd]
  const void* v_new;
  const void* k_pages;      // [pages][nkv][LLG_PAGE][hd]
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* tiles;         // [n_tiles][2]: (sequence index in the batch, first query among its step tokens)
  const int* cu_tokens;     // [B + 1]
  const int* len_before;    // [B]
  const int* slots;         // [B]
  void* out;                // [n_tokens][nh * hd]
  int n_tiles, nh, nkv, hd;
  float scale;
  int window;               // 0 = all keys
  int n_tokens, n_pages;    // rows of k_new / v_new, pages of k_pages / v_pages
  // Further forms of attention; all zero gives the plain one.  Only the kernels of attention_simt.cu and attention_mma.cu
  // read these (a caller checks with the library's *_supported function before it sets them for another kernel).
  int vd;                   // elements of a value head (v_new, v_pages and out then have vd where they say hd); 0 = hd
  int has_sink;             // 1: a sink of score sink_score joins every softmax's denominator and carries no value
  float sink_score;
  const float* gate;        // [n_tokens][nh] or null: a head's output is multiplied by its token's gate
  const float* sinks;       // [nh] or null: with has_sink, query head h's sink has the score sinks[h] instead of sink_score
  int chunked;              // 1: `window` is a chunk size: a query at position p sees the keys from (p / window) * window
                            // on (its own chunk, counted from position 0) instead of the last `window` keys
};

// Attention of one new token per sequence, split kernels (attention_simt.cu, attention_mma.cu).
struct DecodeArgs {
  const void* q;            // [B][nh][hd]
  const void* k_pages;
  const void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* slots;         // [B]
  const int* len_before;    // [B]; the new token's key is already in the cache at this position
  float* part_o;            // [B][nh][n_splits][hd]  un-normalised
  float* part_ml;           // [B][nh][n_splits][2]   running maximum, sum
  int n_seqs, nh, nkv, hd, n_splits;
  float scale;
  int window;
  int vd;                   // as in PrefillArgs; part_o then is [B][nh][n_splits][vd]
  int has_sink;
  float sink_score;
  const float* gate;        // [B][nh] or null
  const float* sinks;       // as in PrefillArgs
  int chunked;
};

// Attention of one new token per sequence, TMA kernel (attention_decode_tma.cu).
struct DecodeTmaArgs {
  const void* q;              // [n_seqs][nh][hd]
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* slots;
  const int* len_before;
  float* part;                // [part_slots][G][hd + PART_PAD]
  int* counters;              // [n_seqs][nh], zero
  void* out;                  // [n_seqs][nh * hd]
  int n_seqs, nh, nkv, hd;
  float scale;
  int window;
  int has_sink;               // as in PrefillArgs (value heads have the key heads' size here)
  float sink_score;
  const float* gate;          // [n_seqs][nh] or null
  const float* sinks;         // as in PrefillArgs
  int chunked;
};

// Residual kept as several streams (hyper-connections), elementwise.cu: hc_add_rmsnorm.  For output row j (token
// r = rows ? rows[j] : j), with S streams X_s of width `hidden`:
//   y = sum of the branch's partials                        (when there is a branch)
//   X_t <- sum_s mix[s][t] X_s + write[t] * y               (all streams at once from the old ones; written back)
//   u = sum_s read[s] X_s   (read == null: the plain sum)
//   out[j] = u / sqrt(mean(u^2) + eps) * weight
// The streams, the small vectors and all sums are float32.
struct HyperNormArgs {
  float* streams;             // [S][n_tokens][hidden]
  long long stream_stride;    // elements between streams
  int n_streams;
  const float* branch;        // [n_partials][n_tokens][hidden] or null
  int n_partials;
  long long partial_stride;
  const float* mix;           // [S][S], indexed [from][to]; with a branch
  const float* write;         // [S]; with a branch
  const float* read;          // [S] or null
  const void* weight;         // [hidden]
  int weight_dtype;
  float eps;
  void* out;                  // [n_out][hidden]
  int out_dtype;
  const int* rows;            // [n_out] or null
  int n_out, hidden;
};

// Preparation of queries, keys, values and head gates from one product's row (elementwise.cu: qkv_row_prep).  A row
// of the product holds q [nh * hd], k [nkv * hd], v [nkv * vd] and, with gates, one more number per query head.  Per
// token: partial sums added, biases added, then an RMS norm over the WHOLE q part and one over the whole k part (each
// with a weight vector of the part's size; null = none); q, k and v are written as qk_prep writes them (packed and/or
// into the cache pages) and the gates as sigmoid(g) in float32.
struct QkvRowPrepArgs {
  const float* qkvg;          // [n_partials][n_tokens][row]
  int n_partials;
  long long partial_stride;
  const void* bias;           // [nh * hd + nkv * hd + nkv * vd] or null (the gates have none)
  const void* q_norm_w;       // [nh * hd] or null
  const void* k_norm_w;       // [nkv * hd] or null
  int w_dtype;                // of bias and norm weights
  float norm_eps;
  const int* positions;       // [n_tokens]
  void* q_out;                // [n_tokens][nh][hd]
  void* k_new;                // [n_tokens][nkv][hd] or null
  void* v_new;                // [n_tokens][nkv][vd] or null
  void* k_pages;              // paged store or null
  void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* seq_of_token;
  const int* slots;
  float* gate_out;            // [n_tokens][nh] or null (the row then has no gate part)
  int n_tokens, nh, nkv, hd, vd;
};

// Layer norm fused with the residual add (layernorm.cu).  For output row j (token r = rows ? rows[j] : j):
//   v = residual[r] + scale * (sum over all given sets of partials)      (written back when there are any)
//   out[j] = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * weight + bias
// Up to LLG_LN_BRANCHES sets of partials (sublayers that ran side by side on the same norm's output).
#define LLG_LN_BRANCHES 4
struct LayerNormArgs {
  float* residual;            // [n_tokens][hidden]
  const float* branch[LLG_LN_BRANCHES];   // each [n_partials[i]][n_tokens][hidden] or null
  int n_partials[LLG_LN_BRANCHES];
  long long partial_stride;   // elements between partials (n_tokens * hidden)
  float scale;
  const void* weight;         // [hidden]
  const void* bias;           // [hidden]
  int w_dtype;
  float eps;
  void* out;                  // [n_out][hidden]
  int out_dtype;
  const int* rows;            // [n_out] or null
  int n_out, hidden;
};

// RMS norm in groups fused with the residual add, the add optionally through a gate and a norm of its own
// (groupnorm.cu).  For output row j (token r = rows ? rows[j] : j), with y = the sum of branch's partials:
//   y *= sigmoid(sum of gate's partials + gate_bias)          where gate is given
//   y  = group_rms(y, post_groups, post_eps) * post_w         where post_w is given
//   v  = residual[r] + y                                      (written back where branch is given)
//   out[j] = group_rms(v, groups, eps) * weight
// group_rms(v, g, e): v in g equal consecutive parts, each divided by sqrt(mean(part^2) + e).
#define LLG_NORM_MAX_GROUPS 65536
struct GroupNormArgs {
  float* residual;            // [n_tokens][hidden]
  const float* branch;        // [n_partials][n_tokens][hidden] or null
  int n_partials;
  const float* gate;          // [gate_partials][n_tokens][hidden] or null
  int gate_partials;
  long long partial_stride;   // elements between partials of either (n_tokens * hidden)
  const float* gate_bias;     // [hidden] or null
  const void* post_w;         // [hidden] or null, stored as weight is
  int post_groups;
  float post_eps;
  const void* weight;         // [hidden]
  int w_dtype;
  int groups;
  float eps;
  void* out;                  // [n_out][hidden]
  int out_dtype;
  const int* rows;            // [n_out] or null
  int n_out, hidden;
};

// The minGRU recurrence over a step's sequences (recurrent.cu).  Row n of the input product holds z | u | g arguments
// (3 * size columns); per channel S_t = (1 - z_t) S_{t-1} + z_t c_t with z = sigmoid(. + bias[0..size)), u = . +
// bias[size..2 size), c = u + 1/2 (u >= 0) or sigmoid(u); out[n] = S_t * silu(g).  state[slot] holds S before the step's
// first token and receives S after its last.  A step whose longest sequence brings more than LLG_MINGRU_PIECE tokens is
// scanned in pieces of that many (the recurrence is linear in S): carry [n_seqs][pieces][2][size] receives every
// piece's (product of 1 - z, state reached from zero); a second kernel walks a sequence's pieces from its state, leaves
// each piece's starting state in the second field and the last state in state[slot]; the scan then runs again, every
// piece from its own starting state, and writes the outputs.  Without carry one kernel does it all.
#define LLG_MINGRU_PIECE 64
struct MinGruArgs {
  const float* rows;          // [n_partials][n_tokens][3 * size]
  int n_partials;
  long long partial_stride;
  const float* bias;          // [2 * size]
  float* state;               // [slots][size]
  const int* slots;           // [n_seqs]
  const int* cu_tokens;       // [n_seqs + 1]
  void* out;                  // [n_tokens][size]
  int out_dtype;
  float* carry;               // or null: no sequence brings more than one piece
  int pieces;                 // pieces per sequence in carry
  int n_seqs, n_tokens, size;
};

// How a router turns logits into a token's experts and their weights (moe.cu).
//   score 0: the `top` largest logits, weights = softmax over them.
//   score 1: s = sigmoid(logit); with groups > 0 the experts form that many equal groups of neighbours, a group's
//            score is the sum of its group_top largest s, and only experts of the keep_groups best groups are eligible;
//            the `top` eligible experts of largest s, weights = s / (sum of the chosen s + sum_eps) * scale.
struct RouterRule {
  int score;
  int groups, keep_groups, group_top;
  float scale, sum_eps;
};

// Preparation for latent attention (latent.cu: latent_prep).  A row of the input product holds, per token, up to three
// runs of columns, each at a column of its own (negative: the run is absent and its part of the work is left out):
// at q_col nh * (dim + rdim) query elements (head by head: dim unrotated, rdim rotated); at kv_col `rank` latent
// elements, then rdim elements of the key part that all heads share; at cq_col cq_rank elements of a latent of the
// queries, which is RMS-normed with cq_norm_w and written to cq_out for the product that makes the queries from it.
// Other columns of the row (row_width in all) are someone else's.
struct LatentPrepArgs {
  const float* rows;          // [n_partials][n_tokens][row_width]
  int n_partials;
  long long partial_stride;
  int row_width, q_col, kv_col, cq_col, cq_rank;
  const void* cq_norm_w;      // [cq_rank], stored as c_norm_w is
  void* cq_out;               // [n_tokens][cq_rank], in the output type
  int pairing;                // which elements a rotation pairs: 0 (i, i + rdim/2), 1 (2i, 2i+1)
  const void* c_norm_w;       // [rank]
  int w_dtype;
  float norm_eps;
  const float* cos_table;     // [positions][rdim / 2] or null (rdim == 0)
  const float* sin_table;
  int table_positions;
  const int* positions;       // [n_tokens]
  void* q_plain;              // [n_tokens][nh][dim]
  void* q_out;                // [n_tokens][nh][rank + rdim]; only the last rdim of every head are written here
  void* k_new;                // [n_tokens][1][rank + rdim] or null
  void* v_new;                // [n_tokens][1][rank] or null
  void* k_pages;              // paged store or null
  void* v_pages;
  const int* page_table;
  int table_width;
  int ring_pages;
  const int* seq_of_token;
  const int* slots;
  int n_tokens, nh, dim, rdim, rank;
};

// y[n][h][o] = sum_k w[h][o][k] x[n][h][k] (latent.cu: head_linear).  x and y may be parts of wider rows: their
// strides between tokens and between heads are given in elements; the innermost elements are contiguous.
struct HeadLinearArgs {
  const void* x;
  long long x_token_stride, x_head_stride;
  const void* w;              // [nh][n_out][n_in]
  void* y;
  long long y_token_stride, y_head_stride;
  int n_tokens, nh, n_in, n_out;
};

// Mixture of experts (moe.cu).  The step's (token, choice) pairs are laid out as rows in the order of their experts, every
// expert's run filled up to whole tiles of `tile` rows (LLG_MOE_TILE for the kernels of moe.cu, 128 for the grouped tcgen05
// product): row_of_pair[p] is pair p's row, token_of_row[r] the token whose activations row r reads (-1: a filling row),
// tile_expert[t] the expert of tile t's rows (-1: an unused tile).
#define LLG_MOE_TILE 32
#define LLG_MOE_MAX_EXPERTS 1024
#define LLG_MOE_MAX_TOP 32

// y[r][o] = sum_k w[e][o][k] x[src(r)][k] for every row r of every tile with an expert e; GATED: two matrices per expert
// and y = silu(w . x) * (w2 . x).
struct GroupedLinearArgs {
  const void* x;              // [.][n_in]; row src(r) = token_of_row ? token_of_row[r] : r
  const int* token_of_row;    // [rows] or null
  const int* tile_expert;     // [rows / LLG_MOE_TILE]
  const void* w;              // [experts][n_out][n_in]
  const void* w2;             // the same shape, or null
  void* y;                    // [rows][n_out]
  int rows, n_in, n_out;
  // Only the tensor-core kernel reads the rest; all zero gives the layout above.  They let it serve a product with one
  // matrix per head over parts of wider rows: without tile_expert the group is the grid's z index and the rows are the
  // n_rows tokens themselves.
  long long x_row_stride, y_row_stride;       // elements between rows (0: n_in, n_out)
  long long x_group_stride, y_group_stride;   // elements by which group e's rows are shifted in x and y
  int n_rows;                                 // without token_of_row: rows from n_rows on are neither read nor written (0: all are)
  long long w_group_stride;                   // elements between the groups' matrices in w and w2 (0: n_out * n_in)
};
