// C interface of the kernel library.  Every function returns 0 on success; otherwise it
// has launched nothing (or reports a failed launch) and rdl_last_error() gives the reason.
// Pointers are device pointers unless said otherwise; `stream` is a cudaStream_t.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RDL_ACT_GELU_TANH 0
#define RDL_ACT_SILU 1

#define RDL_ABI_VERSION 11

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
int rdl_residual_add(void* res_f32, const void* x, int x_dtype, long long total, void* stream);
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
