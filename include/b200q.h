/* b200q -- C ABI of the B200 (sm_100a) quantized-LLM inference kernels.
 *
 * Drop-in boundary for tinygrad's quantized-LLM hot path.  File:line citations
 * are paths inside the tinygrad source tree.  Every pointer named "device" is a
 * raw CUDA device address (for a tinygrad Tensor: `t.uop.buffer.ensure_allocated()._buf`,
 * tinygrad/device.py:128); the library never allocates or frees user-visible
 * memory on the compute entry points.  `stream` is a `cudaStream_t` / `CUstream`
 * passed as `void*` (NULL = the legacy default stream tinygrad's CUDA backend
 * launches on, tinygrad/runtime/ops_cuda.py:65).  Every function returns
 * B200Q_OK (0) or a negative B200Q_ERR_* code, never aborts, and never traps
 * the device; `b200q_strerror` turns the code into text, as the reference turns
 * a CUDA status into a RuntimeError (tinygrad/runtime/ops_cuda.py:13-16).
 */
#ifndef B200Q_H
#define B200Q_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define B200Q_OK 0
#define B200Q_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, unknown enum */
#define B200Q_ERR_BAD_SHAPE (-2)    /* size not a multiple of the quant block / limit exceeded */
#define B200Q_ERR_MISALIGNED (-3)   /* pointer not 16-byte aligned where the kernel needs it */
#define B200Q_ERR_UNSUPPORTED (-4)  /* quant type / dtype combination not built */
#define B200Q_ERR_CUDA (-5)         /* a CUDA call failed: see b200q_last_cuda_error() */
#define B200Q_ERR_TOO_LARGE (-6)    /* request exceeds a fixed capacity of the library */

/* ---- enums -------------------------------------------------------------- */
/* GGML tensor types, numbered as in the GGUF file format (tinygrad/llm/gguf.py:20-21). */
#define B200Q_Q4_0 2
#define B200Q_Q4_1 3
#define B200Q_Q5_0 6
#define B200Q_Q5_1 7
#define B200Q_Q8_0 8
#define B200Q_Q4_K 12
#define B200Q_Q5_K 13
#define B200Q_Q6_K 14
/* element types of activations / outputs */
#define B200Q_F32 0
#define B200Q_F16 1
#define B200Q_BF16 2
/* GEMV epilogues */
#define B200Q_EPI_LINEAR 0   /* y = W x (+bias) (+residual) */
#define B200Q_EPI_SILU_MUL 1 /* weights packed with b200q_repack(raw0=gate, raw1=up): y = silu(gate x) * (up x) */
#define B200Q_MAX_PEERS 8    /* ranks of one tensor- / expert-parallel group (the GPUs of one node) */
/* launch flags */
#define B200Q_FLAG_PDL 1     /* launch with programmatic dependent launch (overlaps the weight prefetch with the previous kernel) */

const char* b200q_strerror(int code);
/* Device-side status word: 0 = fine, 1 = a bounded wait inside a kernel ran out (the kernel then skipped its
 * remaining work instead of spinning; its output is invalid), 2 = a decode-step kernel was handed a position outside
 * [0, max_context) and skipped its cache / token-table access.  Reads and clears it.  Synchronises the device. */
int b200q_status_read_clear(int* status);
const char* b200q_last_cuda_error(void);
int b200q_version(void);

/* ---- runtime plumbing (so the Python host needs no other CUDA binding) -- */
int b200q_device_count(int* count);
int b200q_set_device(int device);
int b200q_device_props(int device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem);
int b200q_malloc(void** device_ptr, size_t bytes);
int b200q_free(void* device_ptr);
int b200q_host_alloc(void** host_ptr, size_t bytes);              /* pinned host memory */
int b200q_host_free(void* host_ptr);
int b200q_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes, void* stream);
int b200q_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes, void* stream);
int b200q_memcpy_d2d(void* device_dst, const void* device_src, size_t bytes, void* stream);
int b200q_memset(void* device_dst, int value, size_t bytes, void* stream);
int b200q_stream_create(void** stream);
int b200q_stream_destroy(void* stream);
int b200q_stream_synchronize(void* stream);
int b200q_device_synchronize(void);
int b200q_event_create(void** event);
int b200q_event_destroy(void* event);
int b200q_event_record(void* event, void* stream);
int b200q_event_synchronize(void* event);
int b200q_event_elapsed_ms(void* start, void* stop, float* ms);
/* Capture everything launched on `stream` between begin and end into a CUDA graph,
 * the counterpart of the reference's TinyJit -> CUDAGraph replay
 * (tinygrad/engine/jit.py:241-291, tinygrad/runtime/graph/cuda.py:10-70). */
int b200q_graph_begin(void* stream);
int b200q_graph_end(void* stream, void** graph_exec);
int b200q_graph_launch(void* graph_exec, void* stream);
int b200q_graph_destroy(void* graph_exec);

/* ---- GGUF block formats -------------------------------------------------
 * Replaces the lazy dequantisation expression `ggml_data_to_tensor`
 * (tinygrad/llm/gguf.py:23-72; Q4_0 :46, Q4_1 :47-49, Q5_0 / Q5_1 :50-55, Q8_0 :56, Q4_K / Q5_K :57-67, Q6_K :68-72).
 *
 * b200q_dequant_raw: raw GGUF blocks -> n_elems values, fp32 (bit-identical to
 * the reference's fp32 expression) or fp16 (its round-to-nearest-even cast,
 * tinygrad/llm/model.py:376). */
int b200q_dequant_raw(int qtype, const void* device_raw, void* device_out, int64_t n_elems, int out_dtype, void* stream);

/* Packed weight layout used by the GEMV kernels (Q4_0, Q8_0, Q6_K).  A [n_out, n_in]
 * weight (blocks running along n_in, as GGUF stores a Linear weight,
 * tinygrad/llm/gguf.py:148) is re-tiled ONCE at load time, losslessly, into
 * tiles of 16 rows x 128 columns (4 quant blocks per row), ordered
 * [row_tile][column_group].  Inside a tile the 32 lanes of a warp each own one
 * (row, block) pair per 16-byte word, so that a warp-wide 128-bit load reads
 * 512 contiguous bytes, followed by the 64 fp16 block scales of the tile:
 *   Q4_0 tile = 1152 B: [lane l: 16 quant bytes of (row l/4,   block l%4)] x32,
 *                       [lane l: 16 quant bytes of (row l/4+8, block l%4)] x32,
 *                       [entry e=2*(l/4)+h: scales of rows l/4 and l/4+8, blocks 2h and 2h+1] x16 (8 B each)
 *   Q8_0 tile = 2176 B: as above with the 32 quant bytes of a (row, block) pair in two 16-byte halves
 *                       (rows 0-7: halves at +0 and +512; rows 8-15: at +1024 and +1536), then the same scale entries.
 *   Q6_K tile = 1696 B (n_in a multiple of 256; a tile row is half a super-block, tinygrad/llm/gguf.py:68-72):
 *                       [lane l: the low nibbles of (row l/4, block l%4): byte i = element i | element i+16 << 4] x32, the same for rows +8,
 *                       [lane l: 8 bytes of high bit pairs: byte k of word 0 holds elements k, 4+k, 8+k, 12+k at bits 0, 2, 4, 6;
 *                        word 1 the same for elements 16..31] x32, the same for rows +8,
 *                       int8 sub-block scales [16 rows][8], fp16 super-block scales [16 rows]  (106 bytes per row against 105 in the file).
 * The bytes per weight element are exactly the GGUF format's for Q4_0 / Q8_0 (18 or 34 bytes per 32).
 * n_out is padded up to a multiple of 16 and n_in to a multiple of 128 with zero-scale blocks.
 * With raw1 != NULL two matrices of equal shape are interleaved 8 rows at a
 * time (rows 0-7 of each tile from raw0, rows 8-15 from raw1) for the fused
 * SwiGLU epilogue; the packed matrix then has 2*n_out rows. */
size_t b200q_packed_bytes(int qtype, int n_out, int n_in);
int b200q_repack(int qtype, const void* device_raw0, const void* device_raw1, void* device_packed, int n_out, int n_in, void* stream);
/* packed -> row-major [n_out, n_in] fp32/fp16 (same values as b200q_dequant_raw of the original blocks) */
int b200q_dequant_packed(int qtype, const void* device_packed, void* device_out, int n_out, int n_in, int out_dtype, void* stream);

/* ---- weight-dequant-fused linear ----------------------------------------
 * Replaces `Linear.__call__` = x.linear(weight.T, bias) on a GGUF-quantised
 * weight (tinygrad/nn/__init__.py:177, tinygrad/mixin/op.py:1257-1274,
 * dot with fp32 accumulation tinygrad/mixin/op.py:367-392), optionally fused with
 * the RMSNorm in front of it (tinygrad/nn/__init__.py:300-304), the residual add
 * behind it (tinygrad/llm/model.py:149-150) or the SwiGLU product
 * (tinygrad/llm/model.py:137).  One launch; weights are streamed once per
 * activation row.  Activations are quantised on the fly to 15-bit integers with one fp32 scale per 32
 * (error ~3e-5 relative, far inside the 1e-2 tolerance of this path); products and sums inside a block
 * are exact integers, accumulation across blocks is fp32. */
typedef struct b200q_gemv_args {
  int qtype;                /* B200Q_Q4_0 | B200Q_Q8_0 | B200Q_Q6_K (plain linears: EPI_LINEAR, no xq_in; n_in a multiple of 256) */
  int n_out;                /* logical output features (for EPI_SILU_MUL: features of gate == up) */
  int n_in;                 /* input features, multiple of 32 */
  int m;                    /* activation rows (1 at decode) */
  const void* w_packed;     /* device, from b200q_repack, 16-byte aligned */
  const void* x;            /* device [m, n_in], x_dtype */
  int x_dtype;              /* B200Q_F32 | B200Q_F16 */
  int y_dtype;              /* B200Q_F32 | B200Q_F16 */
  const void* norm_weight;  /* device fp16 [n_in] or NULL: y = W (rmsnorm(x) * norm_weight) */
  float norm_eps;
  int epilogue;             /* B200Q_EPI_* */
  const void* bias;         /* device fp16 [n_out] or NULL */
  const void* residual;     /* device fp32 [m, n_out] or NULL, added to the result */
  void* y;                  /* device [m, n_out], y_dtype */
  int flags;                /* B200Q_FLAG_* */
  int max_ctas;             /* 0 = library default (a multiple of the SM count) */
  /* Optional hand-over of quantised activations between consecutive launches (m == 1 only), which takes the
   * activation quantisation off the critical path of the consuming GEMV.  A record is b200q_xq_bytes(n) bytes,
   * 16-byte aligned, opaque to the caller (layout: tinygrad_b200/csrc/actquant.cuh). */
  const void* xq_in;        /* device record of the input row written by an upstream kernel (then `x` is ignored and may be
                               NULL).  If norm_weight is set the record already holds x * norm_weight and ss_in gives the
                               partial sums of squares of x for the RMSNorm scalar. */
  const float* ss_in;       /* device [ss_count] or NULL */
  int ss_count;
  void* xq_out;             /* device record to fill with THIS launch's output row (n_out % 128 == 0), optionally
                               multiplied by xq_out_norm_weight first (the next GEMV's RMSNorm weight, fp16 [n_out]);
                               `y` may then be NULL if nobody needs the fp32 values */
  const void* xq_out_norm_weight;
  float* ss_out;            /* device [n_out / 32] partial sums of squares of the output row, or NULL */
  float residual_scale;     /* the residual is multiplied by this before it is added; 0 means 1.  A row-parallel shard of a
                               tensor-parallel linear adds residual / n_ranks so that the all-reduce of the shards yields
                               W x + residual (tinygrad shards the same linears by axis, examples/llama3.py:233-243) */
  /* Sharded linears without a collective library: with n_peers > 0 the output row (m == 1, EPI_LINEAR, bias and residual as
   * given) is ALSO stored into slot `peer_rank` of a mailbox on every rank, peer_mailboxes[d] being rank d's mailbox (fp32 words
   * [n_peers][n_out], this rank's own included) as mapped into this process (b200q_ipc_open).  b200q_mailbox_reduce on each rank
   * then sums the slots (row-split linear: all-reduce) or copies them out (column-split: all-gather).  `y` may be NULL. */
  void* const* peer_mailboxes;   /* host array [n_peers] of device pointers */
  int n_peers, peer_rank;
  /* xq_out without a constraint on how row tiles are dealt to CTAs: device uint32 [n_out + n_out / 32], the first n_out words the
   * all-ones pattern, the rest zero, set once (the kernel leaves them so).  Without it a CTA takes runs of 2 (4 with the SwiGLU
   * epilogue) consecutive row tiles so that it holds whole blocks of 32 outputs, which loads the grid unevenly; with it tiles go
   * out one by one, every tile leaves its outputs in this row as self-validating words and counts into its block's counter, and
   * the CTA that counts last collects and quantises the block.  Same record either way. */
  void* xq_out_stage;
} b200q_gemv_args;
int b200q_gemv(const b200q_gemv_args* args, void* stream);
size_t b200q_xq_bytes(int n);

/* ---- collectives over peer memory (NVLink), no communication library in the data path ---------------------------------
 * Replaces what the reference expands a sharded reduce into: copies of every shard to every device plus add kernels
 * (`handle_allreduce`, tinygrad/schedule/allreduce.py:6-58, over `CUDAAllocator._transfer`, tinygrad/runtime/ops_cuda.py:88-94).
 * A mailbox is a device buffer of 32-bit words [n_slots][n]; a producer (b200q_gemv with n_peers > 0, running on any rank) stores
 * finished fp32 values into slot = its rank, on every rank; an untouched word holds the all-ones pattern.  The consumer polls
 * the words themselves (each is empty or complete: no flag, no fence) and puts the empty pattern back as it reads, so the same
 * mailbox serves the next step; two collectives in a row must use two different mailboxes.
 * b200q_mailbox_reduce: out[i] = (residual ? residual[i] : 0) + slot 0 [i] + slot 1 [i] + ... in slot order (bit-identical on all ranks).
 *   With n_slots == 1 it is a plain hand-over (all-gather: every rank's producer fills its own part of the one slot).
 *   spin_limit: polls per word before the kernel gives up (0 = default, about a second); on expiry the word counts as 0 and the
 *   status word (b200q_status_read_clear) is set to 1.  The mailbox starts out filled with 0xFF bytes (b200q_memset).
 * b200q_ipc_export / _open / _close: a device allocation (b200q_malloc) made visible to the other processes of the node
 * (cudaIpcGetMemHandle / cudaIpcOpenMemHandle); the 64-byte handle travels by any host channel. */
int b200q_mailbox_reduce(void* mailbox, int n_slots, int n, const float* residual, float* out, int spin_limit, int flags, void* stream);
int b200q_ipc_export(void* device_ptr, void* handle64_out);
int b200q_ipc_open(const void* handle64, void** device_ptr);
int b200q_ipc_close(void* device_ptr);

/* Dense (unquantised) Linear at decode: y[m, n_out] = f(x)[m, n_in] . W[n_out, n_in]^T for a weight stored row-major
 * as fp16, bf16 or fp32 (w_dtype) - the Linears a GGUF file leaves unquantised (router ffn_gate_inp, F16 models).
 * Replaces Linear.__call__ (tinygrad/nn/__init__.py:177) for those; f = optional RMSNorm with norm_weight (fp16 [n_in])
 * as in b200q_gemv; bias fp16 [n_out]; residual / y in y_dtype.  fp32 products and accumulation.  n_in % 8 == 0,
 * min(m, 4) * n_in * 4 <= 200 KiB; the weight is streamed once per 4 rows (decode and router sizes; large m with large
 * n_out belongs to a GEMM).  flags: B200Q_FLAG_PDL. */
int b200q_gemv_dense(const void* w, int w_dtype, int n_out, int n_in, int m, const void* x, int x_dtype, const void* norm_weight,
                     float norm_eps, const void* bias, const void* residual, void* y, int y_dtype, int flags, void* stream);

/* out[i] = silu(gate[i]) * up[i], fp32: the SwiGLU product (tinygrad/llm/model.py:137) behind two separate b200q_gemv_dense calls. */
int b200q_silu_mul(const float* gate, const float* up, float* out, int64_t n, int flags, void* stream);

/* The Linear as tinygrad's own runtime launches it (the in-graph seam, tinygrad/tensor.py:390-396: `Tensor.custom_kernel` with a
 * prebuilt PROGRAM, precedent extra/gemm/moe_gemm.py:30-48).  The kernels b200q_tg_gemv_q4_0 / _q8_0(float* y, const float* x,
 * const uint8_t* w_packed, const int32_t* meta) take pointers only (tinygrad passes one per tensor, tinygrad/runtime/ops_cuda.py:18-24),
 * read meta = {n_out, n_in, m} from the device, use static shared memory, and ship as tinygrad_b200/tg_kernels.cubin; block 256, grid
 * (ceil(ceil(n_out / 16) / 8), m).  This entry launches the same kernels with that geometry from the library (parity tests). */
int b200q_tg_gemv(int qtype, float* y, const float* x, const void* w_packed, const int32_t* meta_dev, int n_out, int m, void* stream);

/* ---- decode-step kernels -------------------------------------------------
 * Token embedding lookup to the fp32 residual stream:
 * `token_embd(tokens).float()` (tinygrad/llm/model.py:359).  The token id is read
 * on the device from tokens[*pos]. */
int b200q_embed(const void* device_table_f16, const int32_t* device_tokens /* [max_context + 1] */, const int32_t* device_pos, float* device_x, int dim,
                int vocab, int max_context, void* xq_out /* optional record for the first GEMV (b200q_gemv_args.xq_in), or NULL */,
                const void* xq_norm_weight /* fp16 [dim], multiplied into the record, or NULL */,
                float* ss_out /* [dim / 32] partial sums of squares, or NULL */, int flags, void* stream);

/* One-token GQA attention with RoPE and KV-cache update:
 * tinygrad/llm/model.py:167-198 for T == 1 (`apply_rope` :29-33, cache store
 * :184-186, scaled_dot_product_attention tinygrad/mixin/rand.py:298-326).
 * qkv holds this token's [q | k | v] projections in fp32.  K and V caches are
 * [n_kv_heads][max_context][head_dim] each, fp16 or fp32.  The context is cut
 * into fixed slices of 64 positions, one CTA per (KV head, slice): `n_split` must be at
 * least b200q_attn_min_split(max_context).  Partial results go through `scratch`
 * (b200q_attn_scratch_bytes, zero-initialised once) and the last CTA of a head merges them. */
typedef struct b200q_attn_args {
  const float* qkv;         /* device [n_heads*head_dim + 2*n_kv_heads*head_dim] */
  void* k_cache;            /* device */
  void* v_cache;            /* device */
  int kv_dtype;             /* B200Q_F16 | B200Q_F32 */
  const float* rope;        /* device [max_context][rope_dim]: cos || sin (tinygrad/llm/model.py:15-19) */
  const int32_t* pos;       /* device scalar: position of this token (= tokens already cached) */
  float* out;               /* device [n_heads*head_dim] fp32 */
  void* scratch;            /* device, b200q_attn_scratch_bytes(), zero-initialised once */
  int n_heads, n_kv_heads, head_dim, rope_dim, max_context, n_split;
  int flags;
  void* xq_out;             /* optional: the output row also as a quantised record for the output projection
                               (b200q_gemv_args.xq_in); needs head_dim == 128 */
} b200q_attn_args;
int b200q_attn_min_split(int max_context);
size_t b200q_attn_scratch_bytes(int n_heads, int n_kv_heads, int head_dim, int n_split);
int b200q_attn_decode(const b200q_attn_args* args, void* stream);
/* The same for `n_seqs` sequences that decode in lock-step (tokens [B, 1]: tinygrad/llm/model.py:366-367 with B > 1), one launch: sequence s
 * reads row s of qkv [n_seqs][(n_heads + 2 n_kv_heads) * head_dim], its own caches [n_seqs][n_kv_heads][max_context][head_dim], its
 * position pos[s], writes row s of out [n_seqs][n_heads * head_dim] and uses scratch + s * b200q_attn_seq_scratch_stride(...)
 * (n_seqs strides, zero-initialised once).  xq_out must be NULL. */
size_t b200q_attn_seq_scratch_stride(int n_heads, int n_kv_heads, int head_dim, int n_split);
int b200q_attn_decode_seqs(const b200q_attn_args* args, int n_seqs, void* stream);

/* b200q_attn_decode for callers that must not allocate device memory (no counterpart in the reference, which
 * always allocates through its own allocator).  Meant for hosts that own all device memory themselves -- a frozen
 * serving pool, an arena planner that replays captured work, code running under stream capture -- and therefore have
 * no scratch buffer to pass.  The scratch lives in a fixed array inside the library image instead
 * (b200q_attn_decode_static_capacity() bytes, 2 MiB, resident on every GPU that loads the library until exit);
 * `args->scratch` is ignored.  Calls whose geometry needs more (b200q_attn_scratch_bytes) return B200Q_ERR_TOO_LARGE.
 * The call performs no cudaMalloc/cudaFree.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current: make that first call outside any stream capture.  All calls on a
 * device share the one array: two calls that may overlap on the GPU (different streams) race and must be ordered by
 * the caller.  Always launched fully stream-ordered (B200Q_FLAG_PDL is ignored). */
size_t b200q_attn_decode_static_capacity(void);
int b200q_attn_decode_static(const b200q_attn_args* args, void* stream);

/* Greedy sampling: tokens[*pos + 1] = argmax(logits) (lowest index on ties), then
 * *pos += 1.  At temperature 0 this is what the Gumbel-max expression of
 * tinygrad/llm/model.py:364 selects.  scratch: b200q_argmax_scratch_bytes(), zeroed once.  tokens has max_context + 1
 * entries; at *pos >= max_context nothing is written and the status word is set to 2. */
size_t b200q_argmax_scratch_bytes(void);
int b200q_argmax_advance(const float* device_logits, int n, int32_t* device_tokens, int32_t* device_pos, int max_context, void* scratch,
                         int flags, void* stream);
/* *pos += 1 (a prompt token whose logits are not needed); stops at max_context like b200q_argmax_advance */
int b200q_advance(int32_t* device_pos, int max_context, int flags, void* stream);

/* ---- one whole decode step as one persistent kernel ------------------------------------------------------------------
 * The forward pass of `Transformer.forward` for one new token (tinygrad/llm/model.py:358-364; per block :144-151,167-198,137)
 * followed by the greedy sample: what the reference replays as a captured CUDA graph of ~13 kernels per block
 * (tinygrad/engine/jit.py:241-291).  One cooperative kernel, one CTA per SM, walks every stage itself: the packed weights of
 * every Linear are dealt to the CTAs as equal contiguous byte ranges and streamed through per-warp rings of bulk-async copies
 * that keep running across the stage boundaries; stages meet at a grid barrier; attention runs on (KV head, 64-position slice)
 * units in between.  Dense llama / qwen2 family only: all Linears (the vocabulary head included) in one of Q4_0 / Q8_0.
 * Reads tokens[*pos]; with_head != 0: logits [vocab] and tokens[*pos + 1] = argmax; *pos += 1.
 * b200q_decode_layer: the device pointers of one block (weights from b200q_repack: q | k | v packed back to back, gate / up
 * interleaved).  The array of them lives in DEVICE memory.
 * workspace: b200q_decode_step_workspace_bytes(args) bytes, 256-byte aligned, zero-filled once before the first step (and
 * again after a step that raised the status word: its counters are then out of step).  It carries state from step to step:
 * one workspace per model instance, steps of one instance stream-ordered.
 * Returns B200Q_ERR_UNSUPPORTED / B200Q_ERR_TOO_LARGE (also from b200q_decode_step_supported, which launches nothing) for shapes
 * this kernel does not take (head_dim not a multiple of 32 or above 128, more than 8 query heads per KV head, ...): the
 * per-launch entry points above cover those. */
typedef struct b200q_decode_layer {
  const void* qkv;          /* packed [q_dim + 2 kv_dim, dim] */
  const void* qkv_bias;     /* fp16 [q_dim + 2 kv_dim] or NULL */
  const void* attn_output;  /* packed [dim, q_dim] */
  const void* gate_up;      /* packed, interleaved, [2 hidden_dim, dim] */
  const void* ffn_down;     /* packed [dim, hidden_dim] */
  const void* attn_norm;    /* fp16 [dim] */
  const void* ffn_norm;     /* fp16 [dim] */
  void* k_cache;            /* [n_kv_heads][max_context][head_dim], kv_dtype */
  void* v_cache;
} b200q_decode_layer;
typedef struct b200q_decode_step_args {
  const b200q_decode_layer* layers;   /* device array [n_layers] */
  int n_layers, qtype, dim, hidden_dim, n_heads, n_kv_heads, head_dim, rope_dim, max_context;
  int vocab;                /* rows of `output` */
  int embd_vocab;           /* rows of token_embd */
  int kv_dtype;             /* B200Q_F16 | B200Q_F32 */
  float norm_eps;
  const void* token_embd;   /* fp16 [embd_vocab, dim] */
  const void* output_norm;  /* fp16 [dim] */
  const void* output;       /* packed [vocab, dim]; may be NULL when with_head == 0 */
  const float* rope;        /* [max_context][rope_dim] cos || sin */
  int32_t* tokens;          /* [max_context + 1] */
  int32_t* pos;             /* scalar */
  float* x;                 /* [dim] residual stream */
  float* qkv;               /* [q_dim + 2 kv_dim] */
  float* attn;              /* [q_dim] */
  float* act;               /* [hidden_dim] */
  float* logits;            /* [vocab] */
  void* workspace;
  size_t workspace_bytes;
  int with_head;
  int profile_stamps;       /* diagnostics, with `profile`: time stamps kept per CTA */
  void* profile;            /* NULL, or device uint64 [number of SMs][profile_stamps]: thread 0 of every CTA stores the global nanosecond
                               timer at the start and, per stage: input staged, tiles multiplied, rows finished, barrier passed (after a QKV
                               stage also: attention done, barrier passed) */
} b200q_decode_step_args;
int b200q_decode_step_supported(const b200q_decode_step_args* args);
size_t b200q_decode_step_workspace_bytes(const b200q_decode_step_args* args);
int b200q_decode_step(const b200q_decode_step_args* args, void* stream);

/* ---- batched / prefill linear on tcgen05 tensor cores --------------------------------
 * C[m, n] fp32 = A[m, k] fp16 x W[n, k]^T fp16 with fp32 accumulation in tensor memory: `Linear.__call__` for more than
 * one activation row (tinygrad/nn/__init__.py:177), as the prefill chunks of tinygrad/llm/model.py:464-481 need it.
 * k % 64 == 0; a and w 16-byte aligned.  b200q_tc_status_read_clear: like b200q_status_read_clear for these kernels. */
int b200q_gemm_f16(const void* a_f16, const void* w_f16, float* c, int m, int n, int k, void* stream);
/* The same contraction with W as packed Q4_0 / Q8_0 tiles (b200q_repack), dequantised to fp16 on the way into shared
 * memory -- bit-identical to the reference's materialised fp16 weight (tinygrad/llm/model.py:376) --, x [m, n_in] fp16 or
 * fp32, y fp32 or fp16.  fp16 x: one MMA pass with the fp16-rounded weight (the reference's fp16-activation numerics).  fp32 x:
 * x and the weight both go in as fp16 hi + lo pairs (three MMA passes), which reproduces the reference's fp32 x times unrounded
 * dequantised weight (tinygrad/codegen/late/coalesce.py:100 elides the fp16 cast there) to about 2^-22.  epilogue B200Q_EPI_LINEAR: y [m, n_out] = result + optional
 * fp16 bias [n_out] + optional residual [m, n_out] in y_dtype (may alias y).  B200Q_EPI_SILU_MUL: W is the interleaved
 * gate/up matrix (n_out = its 2 * hidden rows) and y [m, n_out / 2] = silu(gate) * up (tinygrad/llm/model.py:137); no bias or
 * residual.  The weights are streamed once per 128 activation rows: the prefill / batched counterpart of b200q_gemv.
 * x rows must be 16-byte aligned (any n_in % 32 == 0 is). */
int b200q_qgemm(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue, void* y,
                int y_dtype, int m, int n_out, int n_in, void* stream);
/* The same Linear on the pipelined kernel: the activations are first split once into fp16 hi / lo tiles in `workspace`
 * (b200q_qgemm_workspace_bytes(m, n_in) bytes, 16-byte aligned; contents are scratch), which the GEMM's CTAs read by bulk copies while
 * their threads only unpack weights, three 64-column stages in flight.  Same arguments, same numerics (the order of the fp32
 * additions inside the tensor core aside), same epilogues.  Two launches. */
size_t b200q_qgemm_workspace_bytes(int m, int n_in);
int b200q_qgemm_ws(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue, void* y,
                   int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream);
/* The same Linear for a few activation rows (m <= 32: batched decode), the weight-streaming shape: the operands swap roles on the
 * tensor core (weight rows = M, activation rows = N = 32), K is split over CTAs so that every layer fills the GPU, partial sums go
 * through `workspace` (b200q_qgemm_skinny_workspace_bytes) and are added in a fixed order by a second kernel that also applies
 * bias / residual / SwiGLU.  Same operands, numerics and epilogue rules as b200q_qgemm. */
/* The same Linear for a FEW activation rows on the int8 tensor cores (batched decode): the 8 columns of an m16n8k32 MMA are 8 activation
 * rows, so a pass streams the weights once for 8 rows at the one-row GEMV's arithmetic (15-bit activation integers, exact block sums, fp32
 * across blocks); m > 8 takes ceil(m / 8) passes.  Launches per pass: quantise the rows into the MMA's operand order; the streaming
 * kernel, which applies the epilogue itself when n_in <= 4096 and otherwise leaves partial sums per K chunk of 4096 inputs in the
 * workspace; then (n_in > 4096 only) the fixed-order sum with the epilogue.  Arguments as
 * b200q_qgemm_skinny; workspace: b200q_qgemv_rows_workspace_bytes(m, n_out, n_in) bytes, 16-byte aligned. */
size_t b200q_qgemv_rows_workspace_bytes(int m, int n_out, int n_in);
int b200q_qgemv_rows(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue, void* y,
                     int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream);
/* The same with the block's RMSNorm folded into the quantising pre-pass (`self.attn_norm(x)` / `self.ffn_norm(x)` in front of the Linear,
 * tinygrad/llm/model.py:159,167,200): x fp32 [m, n_in] is the un-normed residual stream, norm_weight_f16 [n_in] (NULL: no norm). */
int b200q_qgemv_rows_norm(int qtype, const void* w_packed, const void* x, int x_dtype, const void* norm_weight_f16, float norm_eps, const void* bias_f16,
                          const void* residual, int epilogue, void* y, int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes,
                          void* stream);
size_t b200q_qgemm_skinny_workspace_bytes(int m, int n_out, int n_in);
int b200q_qgemm_skinny(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue, void* y,
                       int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream);
/* ---- prompt processing: the row-wise pieces of Transformer.forward for T > 1 tokens (tinygrad/llm/model.py:358-364,167-198)
 * b200q_embed_rows:   x [n_rows, dim] fp32 = token_embd[tokens[t * token_stride]] (tokens on the device; stride 1: consecutive
 *   positions of one sequence, stride = row length of a [n_seqs, max_context + 1] table: the same position of every sequence); pos_dev (device, may be NULL) is added to the index, so a captured graph follows the position.
 * b200q_rmsnorm_rows: out [n_rows, dim] (out_dtype fp16 / fp32 / bf16) = RMSNorm(x) * weight (tinygrad/nn/__init__.py:300-304).
 * b200q_add_rows_bf16: x[i] += y[i] over n values, x fp32, y bf16 (the residual add behind the bf16 output of the expert FFN).
 * b200q_attn_prefill: qkv [n_rows, (n_heads + 2 n_kv_heads) * head_dim] fp32 holds the projections of the tokens at
 *   positions start_pos .. start_pos + n_rows - 1.  Rotates q and k (half-split RoPE table [max_context, rope_dim] = cos || sin),
 *   appends k / v to the caches [n_kv_heads, max_context, head_dim] (kv_dtype) and writes the causal attention of every new
 *   query over cache rows 0 .. its own position to out [n_rows, n_heads * head_dim] (out_dtype fp16 / fp32).  q_scratch: n_rows * n_heads * head_dim
 *   floats.  Queries and probabilities enter the tensor core as fp16 hi + lo pairs, keys / values as cached.  head_dim in {16, 32, 64, 128}. */
int b200q_embed_rows(const void* table_f16, const int32_t* tokens, int token_stride, const int32_t* pos_dev, int n_rows, int dim, int vocab, float* x,
                     void* stream);
int b200q_rmsnorm_rows(const float* x, const void* weight_f16, float eps, int n_rows, int dim, void* out, int out_dtype, void* stream);
int b200q_add_rows_bf16(float* x, const void* y_bf16, int64_t n, void* stream);
/* x[r, c] += y[r, c] * (gate_logit ? sigmoid(gate_logit[r]) : 1), fp32 [n_rows, dim]: the shared expert of a mixture-of-experts block
 * joining the residual stream, with its optional per-token gate (tinygrad/llm/model.py:131-134). */
int b200q_add_rows_gated(float* x, const float* y, const float* gate_logit, int n_rows, int dim, void* stream);
int b200q_attn_prefill(const float* qkv, void* k_cache, void* v_cache, int kv_dtype, const float* rope, int start_pos, int n_rows, int n_heads,
                       int n_kv_heads, int head_dim, int rope_dim, int max_context, void* q_scratch, void* out, int out_dtype, void* stream);
/* Batched decode (the reference's forward on tokens [B, 1], tinygrad/llm/model.py:358-364 with B > 1): row b of qkv is sequence b's
 * new token, every sequence at position pos (or *pos_dev when that device pointer is given: graph replay); caches
 * [n_seqs, n_kv_heads, max_context, head_dim]; otherwise as b200q_attn_prefill. */
int b200q_attn_decode_batch(const float* qkv, void* k_cache, void* v_cache, int kv_dtype, const float* rope, int pos, const int32_t* pos_dev, int n_seqs, int n_heads,
                            int n_kv_heads, int head_dim, int rope_dim, int max_context, void* q_scratch, void* out, int out_dtype, void* stream);
int b200q_tc_status_read_clear(int* status);

/* ---- MXFP8 mixture-of-experts path --------------------------------------
 * E4M3 values with one E8M0 exponent per 32 along the last axis.
 *
 * b200q_quantize_mxfp8: `quantize_mxfp8` (extra/gemm/cdna_asm_gemm.py:149-159; E4M3 rounding tinygrad/dtype.py:237-260):
 * x [rows, k] (fp32 or bf16) -> q [rows, k] E4M3 codes + e8 [rows, k/32].  With dest_row != NULL the quantised row r is
 * written to the `fan` rows dest_row[r*fan .. r*fan+fan-1] of the outputs instead (= quantise after `dispatch`,
 * extra/gemm/moe_routing.py:124-126; zero the outputs first: a zero row quantises to q = 0, e8 = 0). */
int b200q_quantize_mxfp8(const void* x, int x_dtype, int64_t rows, int k, const int32_t* dest_row, int fan, void* q, void* e8, void* stream);
/* act = silu(gate) * up from h = [gate | up] (bf16 [rows, 2f], the output of the fused gate/up expert GEMM), rounded to
 * bf16 and quantised as above (tinygrad/llm/model.py:129 between the expert GEMMs).  rows_used (device, may be NULL):
 * only the first min(rows, *rows_used) rows are processed; pass off + n_experts to skip the unused tail of the row table. */
int b200q_swiglu_quantize_mxfp8(const void* h_bf16, int64_t rows, const int32_t* rows_used, int f, void* q, void* e8, void* stream);
/* Routing tables (`route`, extra/gemm/moe_routing.py:109-122): topi / weights [n_tokens, k], dest_row [n_tokens*k],
 * off [n_experts+1] (group starts, every group padded to 256 rows).  mode 0: top-k of the logits in descending order,
 * weights = softmax over the k (moe_routing.py:115-116).  mode 1: softmax over all experts, compare-count top-k in
 * ascending order, weights not renormalised (tinygrad/llm/model.py:35-41,118,123-124, the OLMoE defaults).
 * Deterministic (stable counting sort).  scratch: b200q_moe_route_scratch_bytes(). */
size_t b200q_moe_route_scratch_bytes(int n_tokens, int n_experts, int k);
int b200q_moe_rows_max(int n_tokens, int n_experts, int k);   /* m_max_for, extra/gemm/moe_routing.py:89-90 */
int b200q_moe_route(const float* logits, int n_tokens, int n_experts, int k, int mode, int32_t* topi, float* weights, int32_t* dest_row,
                    int32_t* off, void* scratch, void* stream);
/* The same with the group padding as a parameter (pad = 1: compact expert-sorted order, what an expert-parallel sender wants: its
 * rows for one destination rank are one contiguous run) and the per-expert row counts [n_experts] as an optional output. */
int b200q_moe_route_pad(const float* logits, int n_tokens, int n_experts, int k, int mode, int pad, int32_t* topi, float* weights,
                        int32_t* dest_row, int32_t* off, int32_t* counts, void* scratch, void* stream);
/* The gating of tinygrad's own mixture-of-experts block (tinygrad/llm/model.py:110-128): gating = 1 softmax, 2 sigmoid, 3 softmax over
 * the selected logits, 4 sqrt(softplus) (`ExpertGating`, model.py:9-13); sel_bias (fp32 [n_experts] or NULL) is added for the selection
 * only (exp_probs_b); the k experts are listed in ascending order of rank with the lower index winning ties (`pairwise_topk`,
 * model.py:35-41); weights = the scores of the selected experts, renormalised over the k if `normalize`, times `scale`
 * (routed_scaling_factor).  The caller applies the reference's shortcut (softmax + normalize + no bias == gating 3, model.py:116-117).
 * Tables and scratch as b200q_moe_route_pad. */
int b200q_moe_route_gating(const float* logits, const float* sel_bias, int n_tokens, int n_experts, int k, int gating, int normalize, float scale,
                           int pad, int32_t* topi, float* weights, int32_t* dest_row, int32_t* off, int32_t* counts, void* scratch, void* stream);
/* The grouping tables alone, for a selection the caller already has (`ExpertWeights.__call__(sel, x)`, tinygrad/llm/model.py:21-27):
 * topi [n_tokens, k] expert ids (entries outside 0..n_experts-1 must not occur) -> dest_row / off / counts as b200q_moe_route_pad. */
int b200q_moe_route_tables(const int32_t* topi, int n_tokens, int n_experts, int k, int pad, int32_t* dest_row, int32_t* off, int32_t* counts,
                           void* scratch, void* stream);
/* Rows of row_bytes bytes (a multiple of 4) moved through an index table: gather = 0: dst[idx[i]] = src[i]; gather = 1:
 * dst[i] = src[idx[i]]; negative entries are skipped.  The regrouping step on both sides of the expert-parallel exchange
 * (`dispatch` / `combine` across ranks, extra/gemm/moe_routing.py:124-131). */
int b200q_permute_rows(const void* src, const int32_t* idx, int64_t n_rows, int row_bytes, void* dst, int gather, void* stream);
/* `combine` (extra/gemm/moe_routing.py:128-131): out[t] = sum_j weights[t,j] * y[dest_row[t*k+j]], fp32 sum, bf16 in/out. */
int b200q_moe_combine(const void* y_bf16, const int32_t* dest_row, const float* weights, int n_tokens, int k, int d, void* out_bf16, void* stream);
/* `grouped_mx_gemm` (extra/gemm/moe_gemm.py:112-134; kernel contract extra/thunder/amd/grouped_mxfp8_gemm.cpp:32-158):
 * C[m_total, n] bf16 = A_q[m_total, k] x B_q[e][n, k]^T with both operands' E8M0 scales, fp32 accumulation; rows
 * off[e]..off[e+1] use expert e; rows past off[n_experts] are left untouched.  m_total % 256 == n % 256 == k % 128 == 0
 * (the reference's own constraint, moe_gemm.py:120).  Runs on tcgen05 block-scaled MMAs (kind::mxf8f6f4.block_scale).
 * b200q_mx_status_read_clear: like b200q_status_read_clear for this kernel's bounded waits. */
int b200q_mx_status_read_clear(int* status);
/* The gate/up expert GEMM with the activation fused into its epilogue: B holds, per 256 rows, 128 gate rows followed by the 128
 * matching up rows (n = 2 f); instead of C the kernel writes act = silu(gate) * up already quantised, act_q [m_total, f] E4M3 +
 * act_e8 [m_total, f/32] -- the same values as b200q_grouped_mxfp8_gemm followed by b200q_swiglu_quantize_mxfp8 on [gate | up]. */
int b200q_grouped_mxfp8_gemm_swiglu(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                    int m_total, int n, int k, void* act_q, void* act_e8, void* stream);
int b200q_grouped_mxfp8_gemm(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                             int m_total, int n, int k, void* c_bf16, void* stream);
/* The same product with the unrounded fp32 sums as the result (what the per-tensor FP8 linear below scales afterwards). */
int b200q_grouped_mxfp8_gemm_f32(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                 int m_total, int n, int k, float* c_f32, void* stream);

/* ---- per-tensor FP8 linear: `FP8Linear` / `quantize_to_fp8` (extra/fp8/fp8_linear.py:4-16,43-63) ------------------------
 * quantize_to_fp8(x): scale = 448 / (max|x| + 1e-8) over the whole tensor, q = e4m3(clamp(x * scale, +-448)), factor = 1 / scale.
 *   b200q_fp8_absmax: amax (one device float, overwritten) = max|x|;  b200q_fp8_quantize: q [n] E4M3 codes and the factor (one device float).
 * FP8Linear.__call__: y = (x_q . w_q^T with fp32 accumulation) * w_factor * x_factor (+ bias), cast to the activation dtype.  The
 *   contraction is b200q_grouped_mxfp8_gemm_f32 with one group and all E8M0 scale bytes 127 (= 1.0); b200q_fp8_scale_bias is the rest.
 * x / y dtypes: B200Q_F32 | B200Q_F16 | B200Q_BF16; bias fp32 [n] or NULL. */
int b200q_fp8_absmax(const void* x, int x_dtype, int64_t n, float* amax, void* stream);
int b200q_fp8_quantize(const void* x, int x_dtype, int64_t n, const float* amax, void* q, float* factor, void* stream);
int b200q_fp8_scale_bias(const float* acc, int64_t rows, int n, const float* factor_w, const float* factor_x, const float* bias, void* y, int y_dtype,
                         void* stream);

/* ---- expert-parallel exchange over peer memory (NVLink), planned on the device ------------------------------------------
 * `dispatch` / `combine` (extra/gemm/moe_routing.py:124-131) ACROSS ranks: experts split contiguously over the ranks (rank r owns
 * experts r * E / R ...), tokens split over the ranks at the input.  No communication library and no host read in the data path.
 * Per layer and rank, on one stream:
 *   b200q_moe_route_pad(pad = 1)   this rank's tokens over ALL experts, compact expert-sorted order, per-expert counts
 *   b200q_ep_publish_counts        the counts into slot `rank` of every rank's counts mailbox
 *   b200q_ep_plan                  waits for all ranks' counts; send_base[e] = first row, inside the owning rank's grouped buffer, of
 *                                  this rank's rows for expert e (groups padded to 256 rows, sources in rank order -- the placement the
 *                                  single-device `route` gives the concatenated tokens); off_local [E/R + 1] = this rank's group starts
 *   b200q_ep_dispatch              quantises each token row once (E4M3 + E8M0) and stores it into the owners' a_q / a_e8 buffers,
 *                                  records remote_row[t * k + j], then raises "rows landed" on every rank
 *   b200q_ep_wait(which = 0)       consumes the "rows landed" flags of all ranks
 *   b200q_grouped_mxfp8_gemm[_swiglu] x 2 on (a_q, a_e8, off_local, E / R, m_max) -> y [m_max, d] bf16
 *   b200q_ep_signal_results        raises "results ready" on every rank
 *   b200q_ep_wait(which = 1)       consumes the "results ready" flags
 *   b200q_ep_combine               out[t] = sum_j weights[t, j] * y_owner[remote_row[t, j]] pulled from the owners' y buffers
 * The peer-visible buffers (b200q_malloc + b200q_ipc_export / _open) are given as arrays of n_ranks pointers, this rank's own included:
 * counts_all uint32 [n_ranks][n_experts], filled with 0xFF bytes at set-up; flags uint32 [2][n_ranks], zeroed at set-up; a_q / a_e8 /
 * y as the grouped GEMM takes them, m_max rows, zeroed at set-up (rows between the groups are never written).  Waits are bounded; on
 * expiry the kernels carry on with zeros and b200q_mx_status_read_clear reports 1; a plan that does not fit m_max reports 2. */
typedef struct b200q_ep_args {
  int n_ranks, rank, n_experts, k, d_model, n_tokens, m_max;
  const int32_t* topi;       /* routing tables of THIS rank's tokens (b200q_moe_route_pad, pad = 1) */
  const int32_t* dest;
  const int32_t* off;
  const int32_t* counts;
  void* const* counts_all;   /* [n_ranks] pointers, likewise the next four */
  void* const* a_q;
  void* const* a_e8;
  void* const* y;
  void* const* flags;
  int32_t* send_base;        /* [n_experts], written by the plan */
  int32_t* off_local;        /* [n_experts / n_ranks + 1] */
  int32_t* remote_row;       /* [n_tokens * k], written by dispatch */
  void* scratch;             /* 4 zeroed bytes */
} b200q_ep_args;
int b200q_ep_publish_counts(const b200q_ep_args* args, void* stream);
int b200q_ep_plan(const b200q_ep_args* args, void* stream);
int b200q_ep_dispatch(const b200q_ep_args* args, const void* x_bf16, void* stream);
int b200q_ep_wait(const b200q_ep_args* args, int which, int spin_limit, void* stream);
int b200q_ep_signal_results(const b200q_ep_args* args, void* stream);
int b200q_ep_combine(const b200q_ep_args* args, const float* weights, void* out_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif
