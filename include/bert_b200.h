/*
 * bert_b200.h - C ABI of the B200 (sm_100a) BERT encoder plugin kernels.
 *
 * Every entry point below is the drop-in for one C++ free function (or runner method) that the
 * TensorRT-OSS BERT plugins call from their enqueue(); the reference location is cited per
 * function as "ref: <file>:<lines>" with paths relative to the TensorRT-OSS tree.
 *
 * Conventions
 *  - Plain pointers and sizes only. `stream` is a cudaStream_t passed as void*.
 *  - All data pointers are DEVICE pointers unless the name ends in `_host`.
 *  - Functions enqueue work on `stream` and return immediately: they never allocate device
 *    memory, never synchronise and never touch another device (the bert_b200_encoder_*_host
 *    functions are the documented exception: they copy host buffers; _forward_host and
 *    _wait_host block the calling thread).
 *  - Return value: BERT_B200_OK (0) on success, otherwise a bert_b200_status; the reason is
 *    available from bert_b200_last_error() (thread local). Nothing throws, traps, resets the
 *    device or exits the process.
 *  - `type_id` follows nvinfer1::DataType: 0 = FP32, 1 = FP16, 2 = INT8
 *    (ref: include/NvInferRuntimeBase.h:148-160).
 */
#ifndef BERT_B200_H
#define BERT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BERT_B200_API __attribute__((visibility("default")))

/* ref: plugin/common/plugin.h:34-41 (pluginStatus_t) */
typedef enum bert_b200_status
{
    BERT_B200_OK = 0,
    BERT_B200_FAILURE = 1,
    BERT_B200_BAD_PARAM = 2,
    BERT_B200_NOT_SUPPORTED = 3,
    BERT_B200_NOT_INITIALIZED = 4,
    BERT_B200_CUDA_ERROR = 5,
    BERT_B200_DEVICE_TIMEOUT = 6
} bert_b200_status;

enum
{
    BERT_B200_FP32 = 0,
    BERT_B200_FP16 = 1,
    BERT_B200_INT8 = 2
};

/* Library version (major*10000 + minor*100 + patch). */
BERT_B200_API int32_t bert_b200_version(void);
/* Message of the last failure on the calling thread ("" if none). */
BERT_B200_API char const* bert_b200_last_error(void);
/*
 * Bounded device waits (mbarrier / TMEM polling in the tensor-core kernels) give up after a
 * fixed number of polls, record a code in a per-device status word and let the kernel return.
 * This reads (and clears) that word for the current device after synchronising `stream`.
 * 0 = no wait ever expired. The word lives in a buffer the caller supplies per launch
 * (see the `status_word` members below); this helper copies one word device->host.
 */
BERT_B200_API int32_t bert_b200_read_status_word(void const* status_word, void* stream, uint32_t* value_host);

/* ------------------------------------------------------------------------------------------
 * Skip + bias + LayerNorm
 * ------------------------------------------------------------------------------------------ */

/*
 * out = gamma * (x - mean(x)) * rsqrt(var(x) + eps) + beta, x = input + skip (+ bias), row length ld.
 * n = total number of elements (rows = n / ld). type_id 0 or 1; all tensors and parameters in
 * that type. bias may be NULL. Statistics are accumulated in FP32. Any ld % (16 / sizeof(T)) == 0
 * up to 8192 takes the vectorised single-pass kernel; other ld take a scalar kernel.
 * ref: plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:252-286 (computeSkipLayerNorm<T,hasBias>)
 */
BERT_B200_API int32_t bert_b200_skip_layer_norm(void* stream, int32_t type_id, int32_t ld, int64_t n,
    void const* input, void const* skip, void const* beta, void const* gamma, void* output, void const* bias);

/*
 * INT8 in / INT8 out, linear layout: x = dq_scale_in*input + dq_scale_skip*skip (+ bias),
 * out = sat8(rni(LN(x) * q_scale)). beta/gamma/bias are FP16. ld % 16 == 0.
 * ref: plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:219-250 (computeSkipLayerNormDQQ<hasBias>)
 */
BERT_B200_API int32_t bert_b200_skip_layer_norm_dqq(void* stream, int32_t ld, int64_t n, int8_t const* input,
    int8_t const* skip, void const* beta, void const* gamma, int8_t* output, void const* bias, float dq_scale_in,
    float dq_scale_skip, float q_scale);

/*
 * INT8 in / INT8 out on the CHW32-interleaved layout [ld/32][total][32] (no bias).
 * ref: plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelHFace.cu:223-257, 334-359
 *      (launch_large_hface / launch_small_hface)
 */
BERT_B200_API int32_t bert_b200_skip_layer_norm_interleaved_hface(void* stream, int32_t ld, int32_t total,
    int8_t const* input, int8_t const* skip, void const* beta, void const* gamma, int8_t* output,
    float dq_scale_in, float dq_scale_skip, float q_scale);

/*
 * Same plus a second INT8 output `preln` = sat8(rni(x * q_skip_scale)) holding the pre-LN sum.
 * ref: plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelMTron.cu:240-275, 362-410
 *      (launch_large_mtron / launch_small_mtron)
 */
BERT_B200_API int32_t bert_b200_skip_layer_norm_interleaved_mtron(void* stream, int32_t ld, int32_t total,
    int8_t const* input, int8_t const* skip, void const* beta, void const* gamma, int8_t* output,
    int8_t* preln, float dq_scale_in, float dq_scale_skip, float q_scale, float q_skip_scale);

/* ------------------------------------------------------------------------------------------
 * Embedding gather + LayerNorm, mask helpers
 * ------------------------------------------------------------------------------------------ */

/*
 * Fixed-length: ids are [S,B] (S-major: token (s,b) at s*B+b); output [S,B,ld] in type_id
 * (0 or 1); tables in the output type; beta/gamma FP32. LayerNorm without epsilon.
 * A token whose word or segment id lies outside its table produces the row `beta`; pos_emb has pos_size rows and
 * S > pos_size is refused (the reference kernel would read past the table).
 * Extension (not in the reference): if out_i8 != NULL the normalised row is also written
 * quantised, out_i8 = sat8(rni(y * q_scale)); pass NULL to get the reference behaviour.
 * ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:237-252 (embSkipLayerNorm<T>)
 */
BERT_B200_API int32_t bert_b200_emb_layer_norm(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S,
    int32_t const* input_ids, int32_t const* token_ids, float const* beta, float const* gamma,
    void const* word_emb, void const* pos_emb, void const* tok_emb, int32_t word_size, int32_t tok_size,
    int32_t pos_size, void* output, int8_t* out_i8, float q_scale);

/*
 * The same launch also writes the second output of the fixed-length embedding plugin: mask_idx[b] = index of the first 0
 * in column b of the [S,B] int32 `mask`, S if there is none (one warp per sequence after its share of the rows; no
 * second kernel). mask and mask_idx NULL: exactly bert_b200_emb_layer_norm.
 * ref: plugin/embLayerNormPlugin/embLayerNormPlugin.cpp:251-336 (enqueue: embSkipLayerNorm, then computeMaskIdx)
 */
BERT_B200_API int32_t bert_b200_emb_layer_norm_mask_idx(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S,
    int32_t const* input_ids, int32_t const* token_ids, float const* beta, float const* gamma,
    void const* word_emb, void const* pos_emb, void const* tok_emb, int32_t word_size, int32_t tok_size,
    int32_t pos_size, void* output, int8_t* out_i8, float q_scale, int32_t const* mask, int32_t* mask_idx);

/*
 * Packed variable-length: ids are [total], sequence b owns tokens cu_seqlens[b]..cu_seqlens[b+1];
 * the position row is the index inside the sequence. `skip_out` (may be NULL) receives the
 * pre-LayerNorm sum (the "MTron" second output). `total` = cu_seqlens[B] must be given by the
 * caller (it sizes the grid); S is only an upper bound on the sequence length. A token whose position inside its
 * sequence is not in [0, pos_size) - a sequence longer than the position table, a cu_seqlens that does not start at 0
 * or decreases - produces the row `beta`, like a token with an id outside its table.
 * ref: plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernelHFace.cu:105-118 (embSkipLayerNormHFace<T>)
 *      plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernelMTron.cu:106-118 (embSkipLayerNormMTron<T>)
 */
BERT_B200_API int32_t bert_b200_emb_layer_norm_var_seqlen(void* stream, int32_t type_id, int32_t ld, int32_t B,
    int32_t S, int32_t total, int32_t const* input_ids, int32_t const* token_ids, int32_t const* cu_seqlens,
    float const* beta, float const* gamma, void const* word_emb, void const* pos_emb, void const* tok_emb,
    int32_t word_size, int32_t tok_size, int32_t pos_size, void* output, void* skip_out, int8_t* out_i8, float q_scale);

/*
 * mask_idx[b] = index of the first 0 in column b of the [S,B] int32 mask, S if there is none.
 * ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:159-183 (computeMaskIdx)
 */
BERT_B200_API int32_t bert_b200_compute_mask_idx(void* stream, int32_t S, int32_t B, int32_t const* mask,
    int32_t* mask_idx);

/*
 * Packs the [S,B] mask into the fragment-ownership bit layout of the reference fused attention
 * kernels: [B][ceil(S/(16*warps_m))][warps_m*warps_n*warps_k*32] uint32.
 * ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:87-96 (convertMask)
 */
BERT_B200_API int32_t bert_b200_convert_mask(uint32_t S, uint32_t B, uint32_t warps_m, uint32_t warps_n,
    uint32_t warps_k, int32_t const* input_mask_sb, uint32_t* input_mask_x, void* stream);

/*
 * Recovers lengths[b] (first masked key position, S if none) from a packed mask written by
 * bert_b200_convert_mask; row_words is the uint32 stride between sequences in `packed_mask`.
 * The sm_100a attention kernel consumes lengths, so the QKVToContext plugin converts the packed mask
 * it receives from the embedding plugin with this helper. No counterpart in the reference, whose fused
 * kernels read the packed mask directly (plugin/bertQKVToContextPlugin/mhaRunner.cu:835-860).
 */
BERT_B200_API int32_t bert_b200_packed_mask_to_lengths(void* stream, int32_t S, int32_t B, uint32_t warps_m,
    uint32_t warps_n, uint32_t row_words, uint32_t const* packed_mask, int32_t* lengths);

/*
 * cu_seqlens[0] = 0, cu_seqlens[b+1] = cu_seqlens[b] + lengths[b] (int32, B <= 65536).
 * No counterpart in the reference, where the caller prepares cu_seqlens on the host
 * (plugin/embLayerNormPlugin/embLayerNormVarSeqlenPlugin.cpp:370-396 consumes it as an input).
 */
BERT_B200_API int32_t bert_b200_lengths_to_cu_seqlens(void* stream, int32_t B, int32_t const* lengths,
    int32_t* cu_seqlens);

/* ------------------------------------------------------------------------------------------
 * Fully connected (dense contraction)
 * ------------------------------------------------------------------------------------------ */

enum
{
    BERT_B200_ACT_NONE = 0,
    BERT_B200_ACT_GELU_ERF = 1
};

/*
 * C[m,n] = epilogue( sum_k A[m,k] * Wt[n,k] ).
 *  type_id 1: A, Wt FP16, FP32 accumulation (tcgen05 kind::f16);   out_type_id 1.
 *  type_id 2: A, Wt INT8, INT32 accumulation (tcgen05 kind::i8);   out_type_id 1 or 2.
 *  type_id 0: A, Wt FP32, FP32 SIMT kernel;                        out_type_id 0.
 * epilogue(acc) = quant( act( acc * alpha + bias[n] ) ), bias FP32 or NULL, act per `activation`,
 * quant = sat8(rni(x * out_scale)) when out_type_id == 2, identity otherwise.
 * Wt is the weight matrix stored [n][k] (K contiguous); the reference plugin holds W as [k][n]
 * and the host layer transposes it once at plugin construction.
 * lda/ldc are row strides in elements. FP16/INT8 require k % 16 == 0 (bytes of a row multiple
 * of 16) and 16-byte aligned A/Wt/C.
 * `status_word` (may be NULL) is a device uint32 that receives a non-zero code if a bounded
 * device wait expired.
 * ref: plugin/fcPlugin/fcPlugin.cpp:551-610 (FCPluginDynamic::enqueue -> cublasLtMatmul);
 * bias / activation / quantise are separate TensorRT layers in the reference graph.
 */
typedef struct bert_b200_fc_params
{
    int32_t type_id;
    int32_t out_type_id;
    int64_t m, n, k;
    void const* a;
    int64_t lda;
    void const* wt;
    void* c;
    int64_t ldc;
    float const* bias;
    int32_t activation;
    float alpha;
    float out_scale;
    uint32_t* status_word;
} bert_b200_fc_params;

BERT_B200_API int32_t bert_b200_fc(bert_b200_fc_params const* params, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused multi-head attention
 * ------------------------------------------------------------------------------------------ */

/*
 * O = softmax(Q K^T * scale, keys < len_b) V per (sequence b, head n).
 * Tensor-core kernels (FP16, INT8): head sizes 16, 32, 48, 64 (32, 64 when interleaved); smaller heads ride the
 * 64-wide tiles with the missing channels zero-filled by the TMA unit, which replaces the reference's pad / unpad
 * copies (plugin/bertQKVToContextPlugin/zeroPadding2d.cu:190-204). FP16 takes any sequence length (key blocks are
 * streamed with an online softmax; scale_bmm1 must be positive) and ignores scale_softmax / scale_bmm2; INT8 takes
 * S <= 512 (its quantised probabilities need the whole score row in tensor memory) and is BERT_B200_NOT_SUPPORTED
 * beyond, as in the reference (qkvToContextPlugin.cpp:530). FP32 always, and FP16 with other head sizes, run a SIMT
 * kernel (the reference's unfused runner, mhaRunner.cu:533-601).
 * No attention kernel needs scratch memory: `workspace` is ignored and bert_b200_mha_workspace_size() returns 0 (the
 * reference's unfused runner takes its score matrix from the plugin workspace, qkvToContextPlugin.cpp:430-438).
 *
 * Layouts (ref: plugin/bertQKVToContextPlugin/README.md:26-30, mhaRunner.cu:550-552, 1006, 1171):
 *  - fixed  (cu_seqlens == NULL): qkv [S][B][N][3][d], out [S][B][N][d]; valid keys of sequence b
 *    are [0, mask_idx[b]) (mask_idx == NULL means all S).
 *  - packed (cu_seqlens != NULL): qkv [total][N][3][d], out [total][N][d]; sequence b owns rows
 *    cu_seqlens[b]..cu_seqlens[b+1]; S is the maximum sequence length.
 *  - interleaved != 0 (INT8, packed only): qkv is CHW32 [3][N][d/32][total][32], out [N][d/32][total][32]
 *    (ref: plugin/bertQKVToContextPlugin/qkvToContextInt8InterleavedPlugin.cpp:124-127).
 * type_id 1: FP16 in/out, FP32 softmax, logits scaled by scale_bmm1 (= 1/sqrt(d)).
 * type_id 2: INT8 in/out: logit = (q.k)_i32 * scale_bmm1; P_q = sat8(rni(p * scale_softmax));
 *            out = sat8(rni((P_q.v)_i32 * scale_bmm2))
 *            (ref: plugin/bertQKVToContextPlugin/mhaRunner.cu:1178-1190).
 * type_id 0: FP32 SIMT kernel.
 * Rows of sequences with length 0 get all-zero output.
 * ref: plugin/bertQKVToContextPlugin/mhaRunner.cu:533-601 (UnfusedMHARunner::run), :835-860 and
 *      :1127-1265 (FusedMHARunner*::run -> precompiled kernels).
 */
typedef struct bert_b200_mha_params
{
    int32_t type_id;
    int32_t B;
    int32_t S;
    int32_t num_heads;
    int32_t head_size;
    int32_t total; /* packed: cu_seqlens[B]; fixed: ignored */
    void const* qkv;
    void* out;
    int32_t const* cu_seqlens;
    int32_t const* mask_idx;
    int32_t interleaved;
    float scale_bmm1;
    float scale_softmax;
    float scale_bmm2;
    uint32_t* status_word;
    void* workspace;         /* not used (see bert_b200_mha_workspace_size) */
    int64_t workspace_bytes;
} bert_b200_mha_params;

BERT_B200_API int32_t bert_b200_mha(bert_b200_mha_params const* params, void* stream);

/*
 * The same attention on separate Q, K, V tensors of shape [B][N][S][d] with the output [B][N][S][d] - the operand
 * layout of TensorRT's IAttention layer, to which the reference's README tells users to migrate
 * (plugin/bertQKVToContextPlugin/README.md:43-131). FP16 or INT8, head sizes 16 / 32 / 48 / 64, S <= 512;
 * `kv_lengths` (may be NULL: all S) holds the valid keys per sequence like `mask_idx` above; the three scales as above.
 * ref: none in the plugin library (the migration target is a TensorRT layer, not a plugin).
 */
typedef struct bert_b200_attention_bnsd_params
{
    int32_t type_id;
    int32_t B;
    int32_t S;
    int32_t num_heads;
    int32_t head_size;
    void const* q;
    void const* k;
    void const* v;
    void* out;
    int32_t const* kv_lengths;
    float scale_bmm1;
    float scale_softmax;
    float scale_bmm2;
    uint32_t* status_word;
} bert_b200_attention_bnsd_params;

BERT_B200_API int32_t bert_b200_attention_bnsd(bert_b200_attention_bnsd_params const* params, void* stream);

/* Bytes of scratch memory bert_b200_mha wants in `workspace`: always 0. Kept so that callers written against the
 * reference's runner interface have something to ask. ref: UnfusedMHARunner::getWorkspaceSize (mhaRunner.cu:522). */
BERT_B200_API int64_t bert_b200_mha_workspace_size(bert_b200_mha_params const* params);

/*
 * Self-test of the bounded device wait (no counterpart in the reference, whose kernels assert instead,
 * plugin/vc/checkMacrosPlugin.cpp:95-113): launches one small kernel on `stream` in which the library's own wait
 * routine waits on an mbarrier that nothing arrives at, with `limit_ns` (at most 100 ms) in place of the 2 s the
 * kernels use. The kernel returns by itself; afterwards *status_word (device) holds the wait's code (1) and
 * *completed (device, may be NULL) is 0. Asynchronous like the kernels; the context stays usable.
 */
BERT_B200_API int32_t bert_b200_selftest_wait_expiry(void* stream, int64_t limit_ns, uint32_t* status_word, uint32_t* completed);

/*
 * Measurement helper for roofline denominators (no counterpart in the reference): what the tensor pipes of the
 * current GPU sustain for the MMA shape the FC kernels issue - every SM pair runs `k_blocks` x four
 * tcgen05.mma.cta_group::2 of 256 x 256 x 32 bytes of K (type_id 2: INT8, 1: FP16) on operands resident in shared
 * memory, nothing else running. Launches the probe twice on `stream` (warm-up, measurement), BLOCKS until it has
 * finished and returns tera-operations per second in *tera_ops_host. status_word may be NULL.
 */
BERT_B200_API int32_t bert_b200_probe_mma_rate(void* stream, int32_t type_id, int32_t k_blocks, uint32_t* status_word,
    float* tera_ops_host);

/* ------------------------------------------------------------------------------------------
 * Whole-encoder driver (host layer loop over the kernels above)
 * ------------------------------------------------------------------------------------------ */

/*
 * The reference tree no longer ships the network builder that wired the four plugins into a
 * BERT encoder (demo/BERT was removed, CHANGELOG.md:24); this driver reproduces that wiring:
 *   EmbLayerNorm -> L x [ FC(QKV)+bias -> QKVToContext -> FC(out) -> SkipLayerNorm(+bias)
 *                         -> FC(ffn1)+bias+GELU -> FC(ffn2) -> SkipLayerNorm(+bias) ]
 * Weights are device pointers owned by the caller and must outlive the encoder object.
 */
typedef struct bert_b200_layer_weights
{
    void const* wt_qkv;   /* [3E][E], rows ordered [N][3][d] */
    float const* b_qkv;   /* [3E] */
    void const* wt_out;   /* [E][E] */
    void const* b_out;    /* [E], type of the SkipLayerNorm parameters (FP16) */
    void const* ln1_gamma;
    void const* ln1_beta;
    void const* wt_ffn1;  /* [F][E] */
    float const* b_ffn1;  /* [F] */
    void const* wt_ffn2;  /* [E][F] */
    void const* b_ffn2;   /* [E] */
    void const* ln2_gamma;
    void const* ln2_beta;
    /* INT8 only: per-tensor dequantisation steps (real = int8 * scale) */
    float s_in;    /* layer input */
    float s_wqkv, s_qkv;
    float s_ctx;
    float s_wout, s_attn_out;
    float s_ln1;
    float s_wffn1, s_ffn1;
    float s_wffn2, s_ffn2;
    float s_out;   /* layer output */
} bert_b200_layer_weights;

typedef struct bert_b200_encoder_config
{
    int32_t type_id;      /* 1 = FP16, 2 = INT8 (explicit per-tensor scales) */
    int32_t num_layers;
    int32_t hidden_size;
    int32_t num_heads;
    int32_t ffn_size;
    int32_t vocab_size;
    int32_t max_positions;
    int32_t type_vocab_size;
    float dq_probs;
    /* embedding front end */
    void const* word_emb;  /* FP16 [vocab][E] */
    void const* pos_emb;   /* FP16 [max_positions][E] */
    void const* tok_emb;   /* FP16 [type_vocab][E] */
    float const* emb_gamma;
    float const* emb_beta;
    bert_b200_layer_weights const* layers_host; /* host array [num_layers] */
} bert_b200_encoder_config;

typedef struct bert_b200_encoder bert_b200_encoder;

/* Bytes of device workspace bert_b200_encoder_forward needs for `max_tokens` tokens / `max_batch` sequences. */
BERT_B200_API int64_t bert_b200_encoder_workspace_size(bert_b200_encoder_config const* cfg, int32_t max_tokens,
    int32_t max_batch);
BERT_B200_API int32_t bert_b200_encoder_create(bert_b200_encoder_config const* cfg, bert_b200_encoder** out);
BERT_B200_API int32_t bert_b200_encoder_destroy(bert_b200_encoder* enc);
/* Number of kernels the last forward launched (for accounting). */
BERT_B200_API int32_t bert_b200_encoder_last_launch_count(bert_b200_encoder const* enc);

/*
 * Per-kernel timing: when enabled, every launch of the forward is bracketed by CUDA events on the
 * caller's stream. bert_b200_encoder_read_timing synchronises those events and ADDS, per kernel kind,
 * the elapsed milliseconds and launch counts of the last forward to ms[kind] / launches[kind]
 * (arrays of BERT_B200_KIND_COUNT entries owned by the caller).
 */
enum
{
    BERT_B200_KIND_EMB = 0,
    BERT_B200_KIND_FC = 1,
    BERT_B200_KIND_MHA = 2,
    BERT_B200_KIND_SKIPLN = 3,
    BERT_B200_KIND_OTHER = 4,
    BERT_B200_KIND_COUNT = 5
};
BERT_B200_API int32_t bert_b200_encoder_enable_timing(bert_b200_encoder* enc, int32_t on);
BERT_B200_API int32_t bert_b200_encoder_read_timing(bert_b200_encoder* enc, float* ms, int32_t* launches);

/*
 * Max calibration on the FP16 encoder: runs one packed forward and returns, per layer, the largest
 * magnitude of the eight tensors that carry a scale in INT8 mode, in the order
 * { layer input, qkv, ctx, attention-out projection, ln1 output, ffn1 output, ffn2 output, layer output }
 * into amax_host[num_layers][8]. The dequantisation step of a tensor is amax / 127
 * (ref: tools/pytorch-quantization/pytorch_quantization/calib/max.py and tensor_quant.py:511-556).
 * `amax_dev` is a caller-provided device buffer of num_layers*8 floats. Synchronises the stream.
 */
BERT_B200_API int32_t bert_b200_encoder_calibrate(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens,
    void* workspace, int64_t workspace_bytes, void* output, float* amax_dev, float* amax_host);

/*
 * Packed forward on device buffers: ids/segment ids [total], cu_seqlens [B+1] (device),
 * output FP16 [total][E] (INT8 mode: the last layer's INT8 tensor is dequantised into it).
 * max_seqlen bounds every sequence length (<= 512).
 */
BERT_B200_API int32_t bert_b200_encoder_forward(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens,
    void* workspace, int64_t workspace_bytes, void* output);

/*
 * bert_b200_encoder_forward without a workspace argument. (No counterpart in the reference: its plugins get their
 * scratch from TensorRT's workspace.)
 *
 * Who needs it: callers that are not in a position to allocate device memory at all - code that runs inside
 * someone else's memory budget (a plugin's enqueue(), which may only use what the host framework hands it; a
 * serving loop whose whole device pool belongs to another runtime), or code on a path where a failed or slow
 * cudaMalloc is not acceptable. Such a caller passes only its inputs and the output buffer; the intermediate
 * tensors live in a buffer built into the library image.
 *
 * Limit: that buffer is BERT_B200_STATIC_WORKSPACE_BYTES (16 MiB) and every GPU that loads the library keeps it
 * reserved until the process exits. A call whose bert_b200_encoder_workspace_size(cfg, total, B) exceeds it is
 * rejected with BERT_B200_NOT_SUPPORTED and a message naming both sizes (BERT-large INT8: about 1200 tokens;
 * BERT-base FP16: about 950 tokens); bert_b200_encoder_static_workspace_limit() returns the limit.
 *
 * The call itself allocates nothing: no cudaMalloc / cudaFree, no event or stream creation (it refuses to run
 * while per-kernel timing is enabled for that reason). The first call on each device asks the CUDA runtime for the
 * device address of the built-in buffer (that device must be current); make that first call outside any stream
 * capture. All calls on a device share the one buffer, which still holds the previous call's intermediates: the
 * status word is re-zeroed at the start of every call and everything else is overwritten before it is read, but
 * two calls that overlap on the GPU (different streams, or different encoders) corrupt each other - serialise them.
 * The device address is kept for the life of the process: an application that tears the device's primary context
 * down (cudaDeviceReset) must reload the library before it uses this entry point again.
 */
#define BERT_B200_STATIC_WORKSPACE_BYTES (16ll * 1024 * 1024)
BERT_B200_API int64_t bert_b200_encoder_static_workspace_limit(void);
BERT_B200_API int32_t bert_b200_encoder_forward_static(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens,
    void* output);

/*
 * Same through HOST buffers (pinned or pageable): copies ids / segment ids / cu_seqlens to the
 * device staging area at the head of `workspace`, runs the encoder, copies the FP16 output back
 * into output_host and synchronises `stream`.
 */
BERT_B200_API int32_t bert_b200_encoder_forward_host(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids_host, int32_t const* segment_ids_host,
    int32_t const* cu_seqlens_host, void* workspace, int64_t workspace_bytes, void* output_dev,
    void* output_host);

/*
 * Pipelined form of the host interface for a serving loop: nothing is synchronised. The encoder runs on
 * `stream`; the copy of the FP16 output into output_host runs on `copy_stream` (a different stream) as soon as
 * the encoder has finished, so it overlaps the next call's kernels. `slot` (0 or 1) names one of two
 * (output_dev, output_host) buffer pairs the caller alternates between: a call first makes `stream` wait for
 * the previous copy out of the same slot. bert_b200_encoder_wait_host(enc, slot) blocks the calling thread
 * until that slot's output_host is complete. The host id buffers must stay valid until then; the two events
 * per slot are created by the first call that uses the slot (make it outside stream capture).
 * ref: none - the reference leaves host transfers to the application (samples/common/buffers.h).
 */
BERT_B200_API int32_t bert_b200_encoder_forward_host_async(bert_b200_encoder* enc, void* stream, void* copy_stream,
    int32_t slot, int32_t B, int32_t total, int32_t max_seqlen, int32_t const* input_ids_host,
    int32_t const* segment_ids_host, int32_t const* cu_seqlens_host, void* workspace, int64_t workspace_bytes,
    void* output_dev, void* output_host);
BERT_B200_API int32_t bert_b200_encoder_wait_host(bert_b200_encoder* enc, int32_t slot);

#ifdef __cplusplus
}
#endif
#endif /* BERT_B200_H */
