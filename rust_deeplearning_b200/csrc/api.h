// C interface of the kernel library.  Every function returns 0 on success; otherwise it
// has launched nothing (or reports a failed launch) and rdl_last_error() gives the reason.
// Pointers are device pointers unless said otherwise; `stream` is a cudaStream_t.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RDL_ACT_GELU_TANH 0
#define RDL_ACT_SILU 1
#define RDL_ACT_SWISH_LIMIT 2   // min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1), L a parameter

#define RDL_ABI_VERSION 19

const char* rdl_last_error(void);
int rdl_abi_version(void);
// 1 (the default): the decode-path kernels are launched with programmatic dependent launch, so that a
// kernel's start-up overlaps the end of the kernel before it; 0: ordinary launches.
void rdl_set_programmatic_launch(int on);

// Codes a kernel leaves in the step's status word (an int the host reads after the step).  Each
// kernel that can give up a bounded wait has its own.
#define RDL_FAULT_TOKEN_ID 1           // embed_rows: a token id outside the table (its row is NaN)
#define RDL_FAULT_ATTENTION_DECODE 3   // attention_decode: a page copy did not complete
#define RDL_FAULT_GEMM_TC 4            // gemm_tc, one block a tile: a stage or an accumulator was not handed over
#define RDL_FAULT_ATTENTION_TC 5       // attention_prefill_tc: a tile copy or a product did not complete
#define RDL_FAULT_GEMM_TC_PAIR 6       // gemm_tc, pairs of blocks: as 4
#define RDL_FAULT_GEMM_STREAM 7        // gemm_skinny: a weight copy did not complete

// For tests of the bounded waits: the kernel whose fault code is `code` gives up a wait after `cycles`
// clock cycles instead of about a second, and announces `extra_tx_bytes` more bytes to the barrier of
// its first copy than that copy delivers, so that this one wait cannot complete.  The block then
// records its code and returns normally.  code 0 switches the test off.  Kernels with the codes
// RDL_FAULT_ATTENTION_DECODE and RDL_FAULT_GEMM_STREAM honour it.
void rdl_set_wait_test(int code, long long cycles, int extra_tx_bytes);

// One attention call over a batch of sequences: the new tokens of this step are the queries,
// keys and values come from a paged cache and from the step's own packed rows.
typedef struct {
    int dtype;                 // of q, k, v, cache and out
    int n_tokens, n_seqs;      // query rows, sequences
    int n_heads, n_kv_heads, head_dim;
    float score_scale;         // scores are multiplied by it
    float softcap;             // 0: none
    int window;                // 0: all earlier keys; else keys with p - j < window
    const void* q; long long q_stride;                       // row stride in elements; heads are contiguous
    const void* k_new; const void* v_new; long long kv_stride;
    void* out; long long out_stride;
    const int* tok_seq; const int* tok_pos;                  // [n_tokens] sequence index and absolute position
    const int* seq_start;                                    // [n_seqs + 1] first packed row of each sequence
    const int* seq_past;                                     // [n_seqs] position of each sequence's first new token
    const int* seq_cached;                                   // [n_seqs] keys below this position come from the cache
    const void* k_cache; const void* v_cache;                // [pages][kv heads][page_size][head_dim]
    const int* tables; int table_width, page_size, ring_pages;  // [n_seqs][table_width] page lists
    // prefill kernels: query tiles, 64 rows each
    const int* tile_seq; const int* tile_q0; int n_tiles;
    // decode kernel: keys per split, splits launched per (token, kv head), float scratch
    int keys_per_split, max_splits;
    void* scratch; long long scratch_bytes;
    long long counter_bytes;   // size of the counter area at the start of scratch (rdl_attention_decode_counter_bytes)
    int* status;               // optional: set non-zero when a kernel gives up on a bounded wait
    // decode kernel, optional (new_rows != 0): q, k_new and v_new are this step's rows as the projection left
    // them, one token per sequence; the kernel rotates the query and key heads itself (float tables
    // [position][rotary_dim / 2]; rotary_dim 0: no rotation) and writes the new key and value rows to the cache
    const float* rope_cos; const float* rope_sin; int rotary_dim; int new_rows;
    // optional: one float per query head, a logit without key or value that joins the softmax's denominator
    // (exp(sinks[h]) counts once; it is neither scaled nor capped); NULL: none
    const float* sinks;
    // optional: one float per query head; the weight of a visible key is then sigmoid(score + sigmoid_bias[h]) and
    // the weights are not normalised over the keys (no softmax, no denominator, no sinks); NULL: softmax
    const float* sigmoid_bias;
    // filled in by the launcher: clock cycles after which a wait is given up, and the test's extra bytes
    long long wait_cycles; int test_extra_tx;
} AttentionArgs;

int rdl_attention_plain(const AttentionArgs* a, void* stream);
int rdl_attention_prefill(const AttentionArgs* a, void* stream);
int rdl_attention_decode(const AttentionArgs* a, void* stream);
// prefill attention on tcgen05 tensor cores for sequences that start at position 0 and head sizes that are
// multiples of 64; q, k_new and v_new must be the packed rows of one [tokens, row_width] buffer
int rdl_attention_prefill_tc(const AttentionArgs* a, long long row_width, void* stream);
long long rdl_attention_decode_counter_bytes(int n_tokens, int n_kv_heads);
long long rdl_attention_decode_scratch_bytes(int n_tokens, int n_heads, int n_kv_heads, int head_dim, int max_splits);

int rdl_embed_rows(void* out_f32, const void* table, int table_dtype, const int* ids, float scale,
                   int n_rows, int hidden, int vocab, int* status, void* stream);
int rdl_norm_residual_norm(const void* x, int x_dtype, const int* row_index,
                           const void* w1, int w1_dtype, float eps1, float off1, void* res_f32,
                           const void* w2, int w2_dtype, float eps2, float off2,
                           void* y, int y_dtype, int n_rows, int hidden, void* stream);
int rdl_gated_activation(void* out, const void* gate_up, int dtype, int activation, int n_rows, int inter, void* stream);
int rdl_softcap_inplace(void* z_f32, long long total, float cap, void* stream);
int rdl_scale_inplace(void* z_f32, long long total, float scale, void* stream);
int rdl_residual_add(void* res_f32, const void* x, int x_dtype, long long total, void* stream);
// The sum of a block whose sublayers read one norm, and the norm the next part asks for, in one pass over the rows:
//   res <- res + scale * (a + b + c)     (b, c optional; the branches in branch_dtype, the sum in float, in that order)
//   y   <- res / sqrt(mean(res^2) + eps) * (w + off)   in y_dtype, if y is given
int rdl_add_branches_norm(float* res, const void* a, const void* b, const void* c, int branch_dtype, float scale, const void* w,
                          int w_dtype, float eps, float off, void* y, int y_dtype, int n_rows, int width, void* stream);
int rdl_convert_rows(void* out, int out_dtype, const void* in, int in_dtype, const int* row_index,
                     int n_rows, int width, void* stream);
// A step's batch description from pinned host memory to the device, by a kernel (a copy engine's hand-over costs
// several microseconds between two kernels): dst[i] = src_pinned[i] for n_ints (a multiple of 4) values, except that
// dst[tokens_at + i] = sampled[src_pinned[token_src_at + i]] for i < n_fed when `sampled` (device, int32) is given.
int rdl_upload_batch(int* dst, const int* src_pinned, int n_ints, const int* sampled, int token_src_at, int tokens_at,
                     int n_fed, void* stream);

int rdl_rope_cache(void* qkv, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                   int rotary_dim, const float* cos_table, const float* sin_table,
                   const int* tok_seq, const int* tok_pos, int do_rope, int do_write,
                   void* k_cache, void* v_cache, const int* tables, int table_width, int page_size,
                   int ring_pages, const int* seq_end, void* stream);

// Rotation, a norm of every query and key head, and the cache write, on packed rows whose stride may exceed their
// heads: the first n_heads + 2 n_kv_heads heads of head_dim values each are query, key and value heads.  A query or
// key head is rotated in float (the first rotary_dim values, half-split pairs; do_rope 0: not at all) and then, if
// norm_eps > 0, divided by sqrt(sum of its squares / norm_dim + norm_eps) (norm_dim: the head's size before any zero
// padding); it is rounded once, on the way back into the row and into the cache.
int rdl_rope_norm_cache(void* rows, long long row_stride, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                        int rotary_dim, const float* cos_table, const float* sin_table, const int* tok_seq, const int* tok_pos,
                        int do_rope, float norm_eps, int norm_dim, int do_write, void* k_cache, void* v_cache,
                        const int* tables, int table_width, int page_size, int ring_pages, const int* seq_end, void* stream);

// A norm over the whole query projection and over the whole key projection of a token (all heads at once, a weight
// per column: wq [n_heads * head_dim], wk [n_kv_heads * head_dim], float), BEFORE the rotation, then the rotation and
// the cache write as above:  q <- R(q / sqrt(sum(q^2) / q_count + eps) * wq), k likewise.  q_count, k_count: the
// projections' sizes before any zero padding of their heads.
int rdl_rope_projnorm_cache(void* rows, long long row_stride, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                            int rotary_dim, const float* cos_table, const float* sin_table, const int* tok_seq, const int* tok_pos,
                            int do_rope, const float* wq, const float* wk, float eps, int q_count, int k_count, int do_write,
                            void* k_cache, void* v_cache, const int* tables, int table_width, int page_size, int ring_pages,
                            const int* seq_end, void* stream);

// ---- forms of the residual stream and of gates (csrc/rownorm.cu) ----
// Norm after the sum: res <- norm(alpha * res + branch) with norm(v) = v / sqrt(mean(v^2) + eps) * (w + off), in float;
// y (optional) receives the same rows in y_dtype.
int rdl_postnorm(float* res, const void* branch, int branch_dtype, float alpha, const void* w, int w_dtype, float eps,
                 float off, void* y, int y_dtype, int n_rows, int width, void* stream);
// out = c * (norm(a; wa) + norm(b; wb)), float result; a and b in `dtype`, both norms with eps and offset 0
int rdl_norm_pair(float* out, const void* a, const void* b, int dtype, const void* wa, const void* wb, int w_dtype,
                  float eps, float c, int n_rows, int width, void* stream);
#define RDL_GATE_SIGMOID 0
#define RDL_GATE_SILU 1
// out[t, i] = x[t, i] * gate_act(g[t, i]) for i < width; x, g and out in `dtype`, each with a row stride of its own
int rdl_gate_mul(void* out, long long out_stride, const void* x, long long x_stride, const void* g, long long g_stride,
                 int dtype, int gate_act, int n_rows, int width, void* stream);
// Float rows x [rows][groups * group] normed group by group (v / sqrt(mean(v^2) + eps), times w[column] if w is given),
// times gate_act(g[t, column]) if g is given, written in out_dtype.
// gate_first: the gate multiplies x before the norm (the root mean square is that of the gated values).
int rdl_group_norm_gate(void* out, int out_dtype, const float* x, int n_rows, int groups, int group, const void* w,
                        int w_dtype, float eps, const void* g, long long g_stride, int g_dtype, int gate_act, int gate_first,
                        void* stream);

// ---- rows that look back along their sequence (csrc/seq_state.cu) ----
// normed[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w and mixed[t] = normed[t] + (normed[t - 1] - normed[t]) * shift, element by
// element, in float; the row before a sequence's first row of the step is state[slot] (zeros at position 0), and
// state[slot] is left holding the sequence's last normed row.  x float [rows][width]; state float [slots][width].
int rdl_norm_shift(const float* x, const void* w, int w_dtype, float eps, const void* shift, int shift_dtype, float* state,
                   const int* tok_seq, const int* tok_pos, const int* seq_start, const int* slots, void* normed, void* mixed,
                   int out_dtype, int n_rows, int width, void* stream);
// out[t, c] = act(bias[c] + sum_j w[c, j] in[t - (taps - 1 - j), c]) along each sequence (zeros before its start), the
// sum in float; inputs of earlier steps are state[slot][taps - 1][channels] (float), which is left holding the
// sequence's last taps - 1 inputs.  in: rows with a stride of their own; out dense [rows][channels]; bias optional.
int rdl_short_conv(const void* in, long long in_stride, int dtype, int channels, int taps, const void* w, int w_dtype,
                   const void* bias, int silu, float* state, const int* tok_seq, const int* tok_pos, const int* seq_start,
                   const int* slots, void* out, int n_rows, void* stream);
// res[t, i] += sigmoid(gates[t, i] + bias_a[i]) a[t, i] + sigmoid(gates[t, width + i] + bias_b[i]) (b1[t, i] + b2[t, i]), in float;
// b1 NULL: the first term only; b2 optional
int rdl_gated_residual_add(float* res, const void* gates, long long gates_stride, const void* bias_a, const void* bias_b,
                           int bias_dtype, const void* a, const void* b1, const void* b2, int dtype, int n_rows, int width,
                           void* stream);
#define RDL_UNARY_RELU2 16     // max(x, 0)^2
#define RDL_UNARY_SILU 17
int rdl_activation_inplace(void* x, int dtype, long long total, int act, void* stream);

// ---- recurrences whose decay depends on the token (csrc/recurrence.cu) ----
#define RDL_REC_SSM 0
#define RDL_REC_DELTA 1
typedef struct {
    int dtype;                                  // of the rows
    int mode;
    int n_tokens, n_seqs, n_heads, n_key_heads, dim, vdim;
    const void* rows; long long row_stride;     // v (state space: x) of every head from v_col; state space: B from k_col, C from q_col
    int q_col, k_col, v_col;
    // state space: the raw step sizes [tokens][heads] with a stride of their own, and float parameters per head
    const void* dt_rows; long long dt_stride;
    const float* dt_bias; const float* a_log; const float* d_skip;
    // delta rule: float [tokens][key heads * dim], [tokens][heads * dim], [tokens][heads]
    const float* q_f; const float* k_f; const float* g_f; const float* beta_f;
    const int* tok_pos; const int* seq_start; const int* slots;
    float* state;                               // [slots][heads][dim][vdim]
    float* out;                                 // [tokens][heads * vdim]
} RecurrenceArgs;
int rdl_recurrence_scan(const RecurrenceArgs* a, void* stream);
// The state space form in chunks of 64 tokens on tensor cores (csrc/state_space_chunked.cu): bfloat16 rows, state size and
// head size multiples of 16 (state size up to 128), x, B and C on 16-byte boundaries; three launches; work: float scratch
// of rdl_state_space_chunked_work_bytes bytes.
int rdl_state_space_chunked(const RecurrenceArgs* a, void* work, long long work_bytes, void* stream);
long long rdl_state_space_chunked_work_bytes(int n_tokens, int n_seqs, int n_heads, int dim, int vdim);
// The delta rule eight tokens at a time, in float (csrc/delta_rule_chunked.cu): heads of up to 128 key channels; two launches;
// work: float scratch of rdl_delta_rule_chunked_work_bytes bytes, 16-byte aligned.
int rdl_delta_rule_chunked(const RecurrenceArgs* a, void* work, long long work_bytes, void* stream);
long long rdl_delta_rule_chunked_work_bytes(int n_tokens, int n_seqs, int n_heads, int dim, int vdim);
typedef struct {
    int dtype, bias_dtype;
    int n_tokens, n_heads, n_key_heads, dim;
    const void* rows; long long row_stride; int q_col, k_col;       // q and k of the key heads
    const void* decay_rows; long long decay_stride;                 // raw decay logits [tokens][heads * dim]
    const void* beta_rows; long long beta_stride;                   // raw beta logits [tokens][heads]
    const void* dt_bias; const float* a_log;                        // [heads * dim] (bias_dtype), [heads]
    float q_scale, unit_eps;
    float* q_f; float* k_f; float* g_f; float* beta_f;
} DeltaPrepareArgs;
int rdl_delta_prepare(const DeltaPrepareArgs* a, void* stream);

// ---- linear attention with a fixed decay per head (csrc/decay_attention.cu) ----
// Per sequence and head, S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with S [dim][vdim] in float, kept per
// slot between steps.  q, k and v are read from packed rows; before they enter the recurrence q and k may be rotated
// (the first rot_n values, half-split pairs, float tables), q, k and v may go through SiLU, and k is multiplied by
// k_scale - all in float.
typedef struct {
    int dtype;                                  // of the packed rows
    int n_tokens, n_seqs, n_heads, dim, vdim;
    const void* rows; long long row_stride;
    int q_col, k_col, v_col;                    // heads lie one after another from each column
    int silu;                                   // 1: q, k and v go through SiLU
    float k_scale;
    const float* cos_t; const float* sin_t; int rot_n;    // [positions][rot_n / 2]; rot_n 0: no rotation
    const float* decay;                         // [heads]
    const int* tok_pos;                         // [tokens]; -1 marks a padding row
    const int* seq_start;                       // [seqs + 1]
    const int* slots;                           // [seqs] row of `state` that belongs to each sequence
    float* state;                               // [slots][heads][dim][vdim]
    float* out;                                 // [tokens][heads * vdim]
} DecayAttentionArgs;
// token by token, float throughout: the 32-bit path, single-token steps, and the reference of the chunked kernel
int rdl_decay_attention_scan(const DecayAttentionArgs* a, void* stream);
// bfloat16 rows, many tokens: chunks of 64 tokens on tensor cores, the state in float between chunks.  work: a float
// buffer of rdl_decay_attention_chunks(n_tokens, n_seqs) * n_heads * dim * vdim values (a state per chunk and head).
int rdl_decay_attention_chunks(int n_tokens, int n_seqs);
int rdl_decay_attention_chunked(const DecayAttentionArgs* a, void* work, long long work_bytes, void* stream);

// out[m, n] = sum_k x[m, k] * w[n, k], all float, plain FMA in a fixed order of k
int rdl_gemm_f32(void* out, const void* x, const void* w, int m, int n, int k, void* stream);

// out[m, n] = epilogue(sum_k x[m, k] * w[n, k]) for m <= 16, bfloat16 operands, float accumulation.
// gated: w is [2 n, k] (gate rows, then up rows) and the result is act(gate) * up.
// softcap > 0: cap * tanh(v / cap).  out_dtype: RDL_F32 or RDL_BF16.  status (optional) is set non-zero
// when a block gives up a bounded wait for a copy.
int rdl_gemm_skinny(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                    int gated, int activation, float softcap, int* status, void* stream);

// The norms around a few-row product taken off the step's critical path ("deferred norms").
// A branch of the residual stream h ends in a product P (up to 8 rows, as many columns as the stream is wide)
// and is followed by
//   h' = h + norm1(y)     y = P's result, norm1(y) = y / sqrt(mean(y^2) + eps1) * (w1 + off1)
//   x  = norm2(h')        norm2 likewise with (w2, eps2, off2)
//   z  = x W^T            the next product C.
// Written out: x[k] = s2 (h[k] + s1 a'[k]) (w2[k] + off2) with a' = y (w1 + off1), s1 = 1 / sqrt(mean(y^2) + eps1),
// s2 = 1 / sqrt(mean(h'^2) + eps2) and mean(h'^2) = (sum h^2 + 2 s1 sum h a' + s1^2 sum a'^2) / width.  Hence
//   z = s2 (W ht + s1 W at),   ht = h (w2 + off2),   at = a' (w2 + off2):
// C multiplies the two bfloat16 row blocks ht and at (one operand of 16 rows) as soon as they are there and
// applies the two numbers of each row in its epilogue.  P's epilogue writes a', at and, for every 16 columns,
// the four partial sums; C adds those up in a fixed order, and its blocks form h' and the next ht, a slice
// each.  No kernel stands between P and C, and nothing on the way waits for a whole row.
#define RDL_NORM_BRANCH 1      // the call is P
#define RDL_NORM_DEFERRED 2    // the call is C
typedef struct {
    int mode;
    float* sums;                     // [units of 16 columns][8 rows][4]: sum y^2, sum h^2, sum h a', sum a'^2
    int n_sums;                      // C: the units P had (P: taken from n)
    // P
    const float* residual;           // h [rows][n]
    const void* w1; int w1_dtype; float off1;
    const void* w2; int w2_dtype; float off2;
    void* branch;                    // out: a', bfloat16 [rows][n]
    void* scaled;                    // out: at, bfloat16 [rows][n] (the second half of C's operand)
    // C; its x is bfloat16 [16][k]: rows 0.. ht, and at from row 8 on (from row 4 on with up to 4 rows: the
    // halves then share one 8-row fragment of the tensor-core product)
    float eps1, eps2;
    const void* branch_in;           // a' [rows][k]
    const float* residual_in;        // h [rows][k]
    float* residual_out;             // out, optional: h' [rows][k]; not the buffer of residual_in
    const void* w_next; int w_next_dtype; float off_next;    // optional: (w + off) of the norm h' is asked for next
    void* scaled_next;               // out, optional: h' (w_next + off_next), bfloat16 [rows][k]
    const int* row_index; int n_out; // output row j is the operand's row row_index[j] (NULL: j); n_out <= 8 rows
} DeferredNormArgs;
// rdl_gemm_skinny with m <= 8 and one side of a deferred norm.  P: plain epilogue only (not gated, no soft-cap),
// `out` unused.  C: any epilogue; m counts the rows of each half of the operand.
int rdl_gemm_skinny_norm(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                         int gated, int activation, float softcap, const DeferredNormArgs* norm, int* status, void* stream);
// Rows of a residual stream outside a product: h' = h + s1 a' with s1 from the sums (sums NULL: h' = h), written
// to residual_out (optional; may be residual_in), and scaled = h' (w + off) as bfloat16 (optional).
int rdl_stream_rows(const float* sums, int n_sums, float eps1, const void* branch, const float* residual_in,
                    float* residual_out, const void* w, int w_dtype, float off, void* scaled,
                    int n_rows, int width, void* stream);

// The same product and epilogues for any number of rows on tcgen05 tensor cores (TMA-fed, accumulators in
// tensor memory).  n must be a positive number, k a multiple of 8; status (optional) is set non-zero
// when a block gives up a bounded wait.
int rdl_gemm_tc(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                int gated, int activation, float softcap, int* status, void* stream);

// ---- latent attention (csrc/latent.cu) ----
// One call per layer run and step: rotates the rotated part of every query head (in place, or into
// q_rot_out), norms the latent, rotates the shared key part, leaves [c | kr] in latent_out and (do_write)
// in the cache, whose rows are [kv_rank + rot_dim] wide with one key/value head.
typedef struct {
    int dtype, n_tokens;
    void* rows; long long row_stride;          // the input projection's packed rows
    int q_col, n_heads, dim, rot_dim;          // queries start at q_col: heads x [dim | rot_dim]
    int latent_col, kv_rank;                   // [kv_rank | rot_dim] starts at latent_col; < 0: this layer has none of its own
    const void* norm_w; int norm_w_dtype; float eps;
    const float* cos_t; const float* sin_t;    // [positions][rot_n / 2]
    int rot_n, interleaved;                    // dimensions that rotate (the first rot_n of the rotated part); pairing
    const int* tok_seq; const int* tok_pos;
    void* q_rot_out; long long q_rot_stride; int q_rot_head;   // optional: rotated query parts go to q_rot_out[t][h * q_rot_head ..]
    void* latent_out;                          // [tokens][kv_rank + rot_dim]
    int do_write;
    void* cache; const int* tables; int table_width, page_size, ring_pages; const int* seq_end;
} LatentPrepareArgs;
int rdl_latent_prepare(const LatentPrepareArgs* a, void* stream);
// the cache write alone, from latent_out (a write that had to wait for readers of the rows it overwrites)
int rdl_latent_write(const LatentPrepareArgs* a, void* stream);
// packed [Q | K | V] rows with heads padded to `pad` values, for the ordinary attention kernels
int rdl_latent_assemble(void* out, int dtype, const void* rows, long long row_stride, int q_col, const void* kv,
                        const void* latent, int n_tokens, int n_heads, int dim, int rot_dim, int vdim, int kv_rank,
                        int pad, void* stream);
// out[t, h, :vdim] = in[t, h, :vdim] * sigmoid(g[t, h]), out dense [tokens][heads * vdim]; g_elem: a gate per value,
// sigmoid(g[t, h * vdim + i])
int rdl_gate_heads(void* out, int dtype, const void* in, long long in_stride, int in_head, const void* g, long long g_stride,
                   int n_tokens, int n_heads, int vdim, int g_elem, void* stream);
// a product per head: out[t, h, j] = sum_k w[h, j, k] x[t, h, k], optionally times sigmoid(gate[t, h]) (gate_elem: of
// gate[t, h * n_out + j])
typedef struct {
    int dtype, n_tokens, n_heads, n_out, k;
    const void* x; long long x_stride; int x_head;
    const void* w;                             // [heads][n_out][k]
    void* out; long long out_stride; int out_head;
    const void* gate; long long gate_stride;   // optional
    int gate_elem;
} HeadsLinearArgs;
int rdl_heads_linear(const HeadsLinearArgs* a, void* stream);

// Decode attention of the absorbed form on tensor cores (csrc/latent_decode.cu): q [tokens][heads * width] attends over
// the cached rows [pages][1][page_size][width] (bfloat16) as keys and, in their first kv_rank values, as values; the
// first kv_rank values of every head of out [tokens][heads * width] are written.  n_splits blocks share a token's
// keys (scratch of rdl_latent_decode_scratch_bytes when > 1).  sinks (optional, float [heads]): a logit per head without
// key or value whose exponential joins the softmax's denominator once (not scaled).
long long rdl_latent_decode_scratch_bytes(int n_tokens, int n_heads, int kv_rank, int n_splits);
int rdl_latent_decode(void* out, long long out_stride, const void* q, long long q_stride, const void* cache, const int* tables,
                      int table_width, int page_size, int ring_pages, const int* tok_seq, const int* tok_pos, int n_tokens,
                      int n_heads, int width, int kv_rank, float score_scale, int window, int max_keys, int n_splits,
                      void* scratch, long long scratch_bytes, const float* sinks, void* stream);

// ---- routed feed-forward (csrc/moe.cu) ----
// sel[t, k], sel_w[t, k]: the `top` experts of row t by softmax score + correction, and their softmax scores;
// logits: float work space [rows][experts] (two kernels: the logits, then softmax and choice)
// scoring: RDL_ROUTE_SOFTMAX, or RDL_ROUTE_SIGMOID (every expert's score is sigmoid(logit) by itself)
#define RDL_ROUTE_SOFTMAX 0
// RDL_ROUTE_SOFTMAX_CHOSEN: the choice is by the logits themselves and the weights are the softmax over the chosen
// logits only.  bias (optional, float [experts]) is added to the logits before anything else, in every form.
#define RDL_ROUTE_SIGMOID 1
#define RDL_ROUTE_SOFTMAX_CHOSEN 2
int rdl_moe_route(const void* x, int dtype, const float* w_router, const float* bias, const float* correction, int n_rows,
                  int n_experts, int width, int top, int scoring, int* sel, float* sel_w, float* logits, void* stream);
// mid[(t, k), :] = gated(W_gate[e] x_t, W_up[e] x_t) for e = sel[t, k] < n_real; w_gate_up [n_real][2 ff][width]
// activation >= 16 (RDL_UNARY_*): experts of two matrices, mid = act(W_up[e] x_t) with w_gate_up [n_real][ff][width].
// sel_w (optional): the pair's weight multiplies the expert's input, mid = f(W (sel_w[t, k] x_t)).
int rdl_moe_gate_up(void* mid, int dtype, const void* x, const void* w_gate_up, const int* sel, const float* sel_w, int n_rows,
                    int top, int n_real, int ff, int width, int activation, float act_param, void* stream);
// out[t, :] = sum_k sel_w[t, k] (e_k < n_real ? W_down[e_k] mid[(t, k), :] : x[t, :]); w_down [n_real][width][ff]
int rdl_moe_down_combine(void* out, int dtype, const void* mid, const void* x, const void* w_down, const int* sel,
                         const float* sel_w, int n_rows, int top, int n_real, int ff, int width, void* stream);

// Many rows: every pair with a real expert gets a slot in a buffer sorted by expert, each expert's run padded to whole
// tiles of 128 rows (max_tiles * 128 >= n_pairs + 127 n_real slots): pair_slot[pair] (-1: identity expert),
// slot_pair[slot] (-1: padding), tile_group[tile] (-1: not in use).  Then the rows are gathered (bfloat16, width a
// multiple of 8), multiplied tile by tile (rdl_gemm_tc_grouped) and summed per row with the router's weights.
int rdl_moe_align(const int* sel, int n_pairs, int n_real, int max_tiles, int* pair_slot, int* slot_pair, int* tile_group, void* stream);
// rdl_moe_gather with sel_w: the gathered row is the pair's weight times x[t] (weights on the experts' inputs)
int rdl_moe_gather(void* xs, const void* x, const int* slot_pair, const int* tile_group, const float* sel_w, int max_tiles, int top,
                   int width, void* stream);
int rdl_moe_combine(void* out, const void* y, const void* x, const int* pair_slot, const float* sel_w, int n_rows, int top, int width,
                    void* stream);
int rdl_gemm_tc_grouped(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k, int n_groups,
                        const int* tile_group, int gated, int activation, float act_param, int* status, void* stream);

// sampling over float logits [rows, vocab]
typedef struct {
    float temperature;          // < 1e-7: greedy
    int top_k;                  // 0: off
    float top_p;                // >= 1: off
    float repetition_penalty;   // 1: off
    unsigned long long seed;
} SamplingArgs;
// host_tokens (optional): pinned host memory the kernel writes the tokens to as well
int rdl_sample(int* out_tokens, int* host_tokens, const float* logits, int n_rows, int vocab, const SamplingArgs* params,
               const unsigned long long* row_stream, const int* row_step,
               const int* history, const int* history_start, float* work, void* stream);
// the uniform number in [0, 1) that rdl_sample draws with for (seed, stream id, step); host function
float rdl_sampling_uniform(unsigned long long seed, unsigned long long stream, unsigned long long step);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
int rdl_check_attention_args(const AttentionArgs* a, const char* who);
#endif
