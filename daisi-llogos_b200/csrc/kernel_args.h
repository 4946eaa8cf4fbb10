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
//   score 2: s = softmax over all experts' logits; the `top` experts of largest s, weights as for score 1.
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

// Residual add of several terms, each optionally RMS-normed first, fused with the norm of the sum (addnorm.cu).  For
// output row j (token r = rows[j] or j): for every term t, y = sum of its partials [n_partials][n_tokens][hidden]; with
// norm_w, y = y / sqrt(mean(y^2) + norm_eps) * norm_w; residual[r] += scale * y.  Then every output o receives
// residual[r] / sqrt(mean(residual[r]^2) + eps) * (offset + weight), or, without a weight, the row as it is (a cast).
// Weights are float32.  No terms: the row is only normed.
#define LLG_ADDNORM_TERMS 4
#define LLG_ADDNORM_OUTS 2
struct AddNormTerm {
  const float* data;          // [n_partials][n_tokens][hidden]
  int n_partials;
  const float* norm_w;        // [hidden] or null
  float norm_eps;
  float scale;
};
struct AddNormOut {
  void* out;                  // [n_out][hidden]
  const float* weight;        // [hidden], or null: the unnormed row
  float offset;               // added to the weight (1: a weight that holds its difference from one)
};
struct AddNormArgs {
  float* residual;            // [n_tokens][hidden]
  long long partial_stride;   // n_tokens * hidden
  AddNormTerm terms[LLG_ADDNORM_TERMS];
  int n_terms;
  AddNormOut outs[LLG_ADDNORM_OUTS];
  int n_outs;
  int out_dtype;
  float eps;
  const int* rows;            // [n_out] or null
  int n_out, hidden;
};

// Token embedding times a scale, plus a row of a second table chosen by a hash of the token and the one before it in its
// sequence, then an RMS norm of the sum (addnorm.cu).  Row of the pair table: (prev * mul_prev + token * mul_cur) mod
// buckets; a sequence's first token (position 0) takes row `buckets`.  The token before a step's first token comes from
// last_token[slot], which receives the step's last token of the sequence.  norm_w null: no norm.
struct HashEmbedArgs {
  const void* table;          // [vocab][hidden]
  int table_dtype;
  float scale;
  const void* pair_table;     // [buckets + 1][hidden] or null
  int pair_dtype;
  int buckets;
  long long mul_prev, mul_cur;
  const int* token_ids;       // [n_tokens]
  const int* positions;       // [n_tokens]
  const int* seq_of_token;    // [n_tokens]
  const int* cu_tokens;       // [n_seqs + 1]
  const int* slots;           // [n_seqs]
  int* last_token;            // [slots]
  const float* norm_w;        // [hidden] or null
  float norm_offset, eps;
  float* out;                 // [n_tokens][hidden]
  int n_tokens, vocab, hidden;
};

// out[n][j] = act(sum of the partials rows[.][n][j]) * table[token_ids[n]][col0 + j] (addnorm.cu): a gate from the
// residual times a per-token vector looked up by the token's id.
struct TableGateArgs {
  const float* rows;          // [n_partials][n_tokens][width]
  int n_partials;
  long long partial_stride;
  const void* table;          // [vocab][table_width]
  int table_dtype, table_width, col0;
  const int* token_ids;
  int act;                    // an activation kind of llg_act
  void* out;                  // [n_tokens][width]
  int out_dtype;
  int n_tokens, width, vocab;
};

// A short causal convolution per channel along every sequence of a step (recurrent.cu).  The inputs are `channels`
// columns from col0 of a product's float32 partial sums (plus in_bias); out[n][c] = sum_j weight[c][j] *
// input(position - taps + 1 + j) + bias[c], zeros before a sequence's start.  state[slot] holds the last taps - 1 inputs
// of the sequence before the step and receives those after it.
#define LLG_CONV_MAX_TAPS 16
struct ConvArgs {
  const float* rows;          // [n_partials][n_tokens][row_width]
  int n_partials;
  long long partial_stride;
  int row_width, col0, channels, taps;
  const float* in_bias;       // [channels] or null
  const float* weight;        // [channels][taps]
  const float* bias;          // [channels] or null
  float* state;               // [slots][taps - 1][channels]
  const int* slots;           // [n_seqs]
  const int* cu_tokens;       // [n_seqs + 1]
  const int* seq_of_token;    // [n_tokens]
  const int* len_before;      // [n_seqs]
  float* out;                 // [n_tokens][channels]
  void* out2;                 // or null: the same values once more in out2_dtype
  int out2_dtype;
  int n_seqs, n_tokens;
};

// The real-gated linear recurrent unit over a step's sequences (recurrent.cu).  Per channel c of block b = c / block_width:
// r = sigmoid(gates[n][b][o] + gate_bias[b][o]), i = sigmoid(gates[n][b][block_width + o] + gate_bias[b][block_width + o])
// (o = c % block_width), a = exp(-decay_scale * r * softplus(lam[c])), S_t = a S_{t-1} + sqrt(1 - a^2) * i * u[n][c];
// out[n][c] = S_t * gelu_tanh(y) with y the sum of the partials' column y_col + c plus y_bias[c].  State, carry and
// pieces as in MinGruArgs.
struct RgLruArgs {
  const float* rows;          // [n_partials][n_tokens][row_width]
  int n_partials;
  long long partial_stride;
  int row_width, y_col;
  const float* y_bias;        // [size] or null
  const float* u;             // [n_tokens][size]
  const float* gates;         // [n_tokens][size / block_width][2 * block_width]
  const float* gate_bias;     // [size / block_width][2 * block_width]
  const float* lam;           // [size]
  float decay_scale;
  float* state;               // [slots][size]
  const int* slots;
  const int* cu_tokens;
  void* out;                  // [n_tokens][size]
  int out_dtype;
  float* carry;
  int pieces;
  int n_seqs, n_tokens, size, block_width;
};

// Retention: linear attention with a fixed decay per head and no softmax (recurrent.cu).  A row of the input product holds
// q (nh * dim) at q_col, k (nh * dim) at k_col, v (nh * vdim) at v_col and the output gate's arguments (nh * vdim) at
// g_col.  q and k are rotated by halves over their first rotary_dim elements, k times k_scale; per head
// S_t = decay[h] S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; out[n][h] = o_t / sqrt(mean(o_t^2) + eps) * silu(g).  state[slot] is
// [nh][dim][vdim] float32.  With carry, pieces of a sequence are run side by side from zero, joined, and run again.
#define LLG_RETENTION_PIECE 128
struct RetentionArgs {
  const float* rows;          // [n_partials][n_tokens][row_width]
  int n_partials;
  long long partial_stride;
  int row_width, q_col, k_col, v_col, g_col;
  const float* cos_table;     // [table_positions][rotary_dim / 2] or null
  const float* sin_table;
  int rotary_dim, table_positions;
  const int* positions;       // [n_tokens]
  const float* decay;         // [nh]
  float k_scale, eps;
  float* state;               // [slots][nh][dim][vdim]
  const int* slots;
  const int* cu_tokens;
  void* out;                  // [n_tokens][nh * vdim]
  int out_dtype;
  float* carry;               // [n_seqs][pieces][nh][dim][vdim] or null
  int pieces;
  int n_seqs, n_tokens, nh, dim, vdim;
};
