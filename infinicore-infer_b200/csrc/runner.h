// The native step: a model is a list of launch records that its parts emitted once; a step replays them.
//
// A record (RunnerOp) names one operation of a layer kind: what it reads and writes (buffer slots), its weights and
// its constants.  It does not name a kernel: which kernel runs it depends on the step (how many rows, which precision)
// and is decided here, in one place, by the rules of host_rules.h.  The records know nothing of the model they belong
// to, and this file knows nothing of any architecture: a layer that can be said in these operations runs natively,
// whatever it is part of; what cannot is run by its own code between two runs of records.
// (The reference's counterpart is the hand-written layer loop of inferDeviceBatch, src/models/jiuge/jiuge.cpp:126-305.)
#pragma once

#include <cuda_runtime.h>

#include "host_rules.h"

// ---- entry points of the kernel modules (signatures as in their sources) -------------------------------
extern "C" {
typedef int (*EmbedFn)(const int *, int, const void *, int, int, float, float *, cudaStream_t);
typedef int (*AddRmsnormFn)(float *, const void *, int, float, const float *, float, float, void *, int, const int *, int,
                            int, cudaStream_t);
typedef int (*ResidualAddFn)(float *, const void *, int, float, long long, cudaStream_t);
typedef int (*SwigluFn)(const void *, int, void *, int, int, int, cudaStream_t);
typedef int (*RopeKvFn)(const void *, int, int, const float *, const int *, const int *, const int *, int, int,
                        const float *, const float *, int, void *, void *, void *, int, int, int, int, int, int,
                        cudaStream_t);
typedef int (*GemmF32Fn)(const float *, int, const float *, int, const float *, float *, int, int, int, int, cudaStream_t);
typedef int (*LinearSmallFn)(const void *, const void *, void *, int, int, int, int, int, int, cudaStream_t);
typedef int (*LinearSmallQkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int, cudaStream_t);
typedef int (*GemmTcgen05Fn)(const void *, const void *, void *, int, int, int, int, int, float, int *, int, cudaStream_t);
typedef int (*GemmTcgen05QkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int *, int, cudaStream_t);
typedef int (*AttentionRowsFn)(const void *, const void *, const void *, void *, int, const int *, const int *, const int *, int,
                               int, int, int, int, int, float, int, int, int, const float *, int, float, int, cudaStream_t);
typedef int (*AttentionDecodeFn)(const void *, const void *, const void *, void *, float *, const int *, int, const int *,
                                 const int *, const int *, int, int, int, int, int, float, int, int, int, const float *, int, float, int,
                                 cudaStream_t);
typedef int (*AttentionPrefillFn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, float, int, int, const float *, int, float, int,
                                  cudaStream_t);
typedef int (*AttentionTcgen05Fn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, int, float, int, int *, int, const float *, int,
                                  float, int, cudaStream_t);
typedef int (*SupportsFn)(int, int, int);
typedef int (*LinearSmallPartsFn)(const void *, long long, const int *, int, const void *, void *, int, int, int, int, int, cudaStream_t);
typedef int (*Supports1Fn)(int);
typedef int (*LinearSmallNormFn)(const void *, const void *, void *, int, int, int, int, int, const unsigned long long *, float,
                                 void *, const float *, unsigned long long *, float, int *, int, cudaStream_t);
typedef int (*LinearSmallQkvNormFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                    const int *, const int *, const int *, int, int, int, int, int,
                                    const unsigned long long *, float, int, cudaStream_t);
typedef const char *(*LastErrorFn)();
// csrc/mixers.cu
typedef int (*LayernormFn)(const float *, const int *, int, int, const float *, const float *, float, float *, void *, int, cudaStream_t);
typedef int (*CastRowsFn)(const float *, void *, int, long long, cudaStream_t);
typedef int (*GluFn)(const float *, void *, int, int, int, int, float, cudaStream_t);
typedef int (*ConvQkvFn)(const float *, int, int, int, int, int, int, int, int, int, const float *, const float *, const float *, int,
                         const float *, const float *, float, const float *, int, float *, const int *, const int *, const int *,
                         const int *, const int *, int, int, void *, void *, void *, int, int, int, int, float, int, const float *, cudaStream_t);
typedef int (*LinearScanFn)(const float *, int, int, int, int, int, int, int, int, float, const float *, const void *, int, const float *,
                            int, int, float, float *, const int *, const int *, int, int, float *, const int *, int, const int *, int,
                            const int *, int, float *, long long, int, const float *, int, int, cudaStream_t);
typedef int (*NormGateFn)(const float *, const float *, int, int, const float *, float, int, int, int, int, void *, int, int, cudaStream_t);
typedef int (*TokenShiftFn)(const void *, const float *, float *, const int *, const int *, const int *, void *, int, int, int, int, int,
                            cudaStream_t);
typedef int (*ActRowsFn)(const float *, int, void *, int, int, int, int, cudaStream_t);
// csrc/blocks.cu
typedef int (*NormAddFn)(const float *, float *, const float *, float, const float *, float, void *, int, int, int, cudaStream_t);
typedef int (*ConcatCastFn)(const float *, const float *, void *, int, int, int, cudaStream_t);
typedef int (*AddBiasRowsFn)(float *, const float *, int, int, cudaStream_t);
typedef int (*LatentQkvFn)(const float *, int, int, int, int, int, int, int, int, const float *, float, const float *, float, const int *,
                           const int *, const int *, int, int, void *, void *, void *, int, int, const float *, int, cudaStream_t);
typedef int (*HeadLinearFn)(const void *, const void *, void *, int, int, int, int, int, int, const float *, int, cudaStream_t);
typedef int (*LatentAttentionFn)(const void *, const void *, void *, float *, int, const int *, const int *, const int *, int, int, int,
                                 int, int, int, float, int, const int *, int, int, cudaStream_t);
typedef long long (*LatentScratchFn)(int, int, int, int);
typedef int (*CausalConvFn)(const float *, int, int, int, const float *, const float *, int, int, float *, const int *, const int *,
                            const int *, float *, void *, int, int, int, cudaStream_t);
typedef int (*SelectiveScanFn)(const float *, const float *, int, int, int, int, const float *, int, const void *, const float *,
                               const float *, const float *, float *, const int *, const int *, int, void *, int, float *, int, int,
                               cudaStream_t);
typedef int (*RoutedExpertsFn)(const void *, const float *, const void *, const void *, float *, int, int, int, int, int, int, int, int,
                               int *, void *, float *, int, float, const float *, const float *, cudaStream_t);
typedef long long (*RoutedWorkspaceFn)(int, int, int);
typedef int (*CountFn)();
typedef int (*SoftcapFn)(float *, float, long long, cudaStream_t);
typedef int (*AddRowsFn)(float *, const void *, int, int, const int *, int, int, int, cudaStream_t);
// csrc/mixers.cu
typedef int (*DeltaRuleFn)(const float *, int, int, int, int, const float *, int, int, int, const float *, const float *, int, int, int, int,
                           float, float, float *, const int *, const int *, int, float *, float *, int, cudaStream_t);
typedef long long (*DeltaScratchFn)(int, int, int, int);
typedef int (*ArgmaxFn)(const float *, long long, int, int, int *, void *, cudaStream_t);
typedef int (*SampleFn)(const float *, long long, int, int, const float *, const int *, const float *, const float *, int *,
                        cudaStream_t);
}

struct RunnerFns {
    EmbedFn embed;
    AddRmsnormFn add_rmsnorm;
    ResidualAddFn residual_add;
    SwigluFn swiglu;
    RopeKvFn rope_kv;
    GemmF32Fn gemm_f32;
    LinearSmallFn linear_small;
    LinearSmallQkvFn linear_small_qkv;
    GemmTcgen05Fn gemm_tcgen05;
    GemmTcgen05QkvFn gemm_tcgen05_qkv;
    AttentionRowsFn attention_rows;
    AttentionDecodeFn attention_decode;
    AttentionPrefillFn attention_prefill;
    Supports1Fn attention_prefill_supports;
    AttentionTcgen05Fn attention_tcgen05;
    LastErrorFn err_elementwise, err_linear_small, err_gemm_tcgen05, err_attention, err_attention_tcgen05;
    // products of few rows: what the small-row kernels take, and the tcgen05 kernel with the weights on the MMA's M side
    // (part of the gemm_tcgen05 module: bound with it or not at all)
    SupportsFn linear_small_supports, linear_small_qkv_supports;
    GemmTcgen05Fn gemm_skinny;
    // few-row products of a chain in which RMSNorm has no kernel of its own
    SupportsFn linear_small_norm_supports;
    LinearSmallNormFn linear_small_norm;
    LinearSmallQkvNormFn linear_small_qkv_norm;
    // sampling (used by the C interface only; may be empty for a caller that samples by itself)
    ArgmaxFn argmax;
    SampleFn sample;
    LastErrorFn err_sampling;
    // layer norm, short convolutions, linear-attention recurrences and their companions (csrc/mixers.cu): bound together,
    // and only for a model whose records name them
    LayernormFn layernorm;
    CastRowsFn cast_rows;
    GluFn glu;
    ConvQkvFn conv_qkv;
    LinearScanFn linear_scan;
    NormGateFn norm_gate;
    TokenShiftFn token_shift;
    ActRowsFn act_rows;
    LastErrorFn err_mixers;
    // norms around sublayers, latent attention, selective scans, routed experts (csrc/blocks.cu): bound together, and
    // only for a model whose records name them
    NormAddFn norm_add;
    ConcatCastFn concat_cast;
    AddBiasRowsFn add_bias_rows;
    LatentQkvFn latent_qkv;
    HeadLinearFn head_linear;
    LatentAttentionFn latent_attention;
    LatentScratchFn latent_attention_scratch;
    CausalConvFn causal_conv;
    SelectiveScanFn selective_scan;
    RoutedExpertsFn routed_experts;
    RoutedWorkspaceFn routed_experts_workspace;
    CountFn routed_experts_launches;
    SoftcapFn softcap;
    LastErrorFn err_blocks;
    // several few-row products of one launch (csrc/linear_small.cu); may be empty: the products then run one by one
    LinearSmallPartsFn linear_small_parts;
    SupportsFn linear_small_parts_supports;
    // rows of a table added to the stream (csrc/blocks.cu, bound with that module) and the gated delta rule (csrc/mixers.cu,
    // bound with that one); may be empty for a caller whose records name neither
    AddRowsFn add_rows;
    DeltaRuleFn delta_rule;
    DeltaScratchFn delta_rule_scratch;
};

// ---- records ---------------------------------------------------------------------------------------------------
// Buffers of a step, by slot.  An operation reads and writes slots; the caller says where each slot lies (and how many
// bytes it holds) when it runs the records, so the same records run over the runner's own buffers or over a caller's
// tensors.
enum RunnerSlot {
    SLOT_X = 0,         // float32 [T, hidden]: the residual stream
    SLOT_DELTA,         // float32 [T, hidden]: a product that has not been added to the stream yet
    SLOT_H,             // activations [T, width]: a norm's output, the operand of the next product
    SLOT_Q,             // activations [T, heads * head size]: rotated queries
    SLOT_O,             // activations [T, heads * head size]: attention's output
    SLOT_ACT,           // activations [T, intermediate]: the gated feed-forward's inner activations
    SLOT_HW,            // activations [wanted rows, hidden]: the final norm's output
    SLOT_LOGITS,        // float32 [wanted rows, vocabulary]
    SLOT_TMP,           // float32: the product before an unfused rotation or activation ([T, widest such product])
    SLOT_DECODE,        // float32: partial results of the split-key attention
    SLOT_MIX,           // float32 [T, heads * value size]: a recurrence's output before its norm and gate
    SLOT_SCAN,          // float32: the states and running decays of a recurrence's pieces; a scan's small projections
    SLOT_X0,            // float32 [T, hidden]: the embedding's output, for a model that feeds it in again later
    SLOT_ROUTE,         // int32 and float32: which experts each row chose, and the rows of each expert
    SLOT_SHIFT,         // activations [parts, T, width]: a row mixed with the row before it, once per projection that reads one
    RUNNER_SLOTS
};

enum RunnerOpKind {
    OP_EMBED = 1,       // out[t] = scale * table[tokens[t]]                                         -> float32 stream
    OP_NORM,            // stream += pending; out = out_scale * rmsnorm(stream[rows]) * weight        rows: all | wanted
    OP_QKV,             // [q | k | v] = in w^T (+ bias); rotate q and k; q -> out, k and v -> their pages
    OP_ATTENTION,       // out = softmax(q K^T * scale, causal, window) V over the paged cache
    OP_RESIDUAL,        // stream += scale * (in w^T)   (left pending for the next norm where no kernel adds in place)
    OP_GATE_UP,         // out = silu(in w_gate^T) * (in w_up^T), w = [gate rows; up rows]
    OP_LINEAR,          // out (float32) = in w^T (+ bias)                                            rows: all | wanted
    OP_CAST,            // out = activations(stream): the operand of a sublayer that reads the stream itself
    OP_LAYERNORM,       // in = SLOT_DELTA: stream += LN(in) (and out = activations(stream) if out_slot >= 0);
                        // in = SLOT_X: out = LN(stream[rows])                                        rows: all | wanted
    OP_CONV_QKV,        // in: float32 rows [q | k | v | ...]; short convolution over time, RMS norm over the whole q and k,
                        // partial rotation; q -> out, k and v -> their pages; the convolution's tails move forward
    OP_LINEAR_ATTENTION,// in: float32 rows [q | k | v | gate | ...]; S = diag(a) S + k v^T, o = S^T q per head over each
                        // request's rows and its state slot; out = rmsnorm(o) * w * act(gate)
    OP_NORM_ADD,        // in = SLOT_DELTA: stream += rmsnorm(in) * vec; if out_slot >= 0: out = rmsnorm(stream) * vec2 (the next
                        // sublayer's input; vec2 null: out = activations(stream))
    OP_REINJECT,        // stream = [stream | in] w^T + vec, in = SLOT_X0: the embedding's output fed in again
    OP_LATENT_QKV,      // in: float32 rows [q | latent and shared key part | ...]; the heads' plain query parts -> out2, their
                        // rotated parts -> out (behind the `rank` elements OP_HEAD_LINEAR fills); the normed latent vector and
                        // the rotated key part -> the row's place in the pages
    OP_HEAD_LINEAR,     // out[t, h, 0..n) = in[t, h, 0..k) w[h]^T for every head (w [heads, n, k]), rows of out `out_hs` apart
                        // per head; gated: times sigmoid(SLOT_TMP[t, g_off + h n + j])
    OP_LATENT_ATTENTION,// out[t, h] = softmax(q[t, h] . page rows * scale, causal) (page rows' first `rank` elements)
    OP_CAUSAL_CONV,     // in: float32 rows; n channels at q_off pass `taps` taps over time (+ bias, act); out = activations,
                        // out2 = float32; the request's tails (state) move forward
    OP_SELECTIVE_SCAN,  // in = x [T, n] float32, in2 = [dt part (rank) | B (k) | C (k)] float32, z = SLOT_TMP[t, g_off + c]; the n
                        // columns of SLOT_TMP at q_off (the in-projection's x part, dead by now) take the step sizes of long steps;
                        // S = exp(dt A) S + dt x B, y = S C + D x over each request's rows and its state slot; out = y silu(z)
    OP_EXPERTS,         // SLOT_DELTA (+)= sum over each row's `top` experts of largest sigmoid(vec in) of expert(score * in)
    OP_SOFTCAP,         // logits = cap * tanh(logits / cap) over the wanted rows
    OP_TOKEN_SHIFT,     // out[s, t] = in[t] + (in[t - 1] - in[t]) * vec[s] for s < heads (the parts), vec [parts, n]; the row before a
                        // portion's first row is kept in state [slots, n]
    OP_ACTIVATE,        // out = activations(act(in)), in: float32 rows `ld` apart, n columns: the unit between the two products of a
                        // feed-forward without a gate
    OP_ADD_ROWS,        // stream[t] += w[positions[t]] (fixed_row < 0) or w[fixed_row]: learned position vectors, a vector per pass;
                        // w [k, n] of type w_dtype
    OP_DELTA_RULE,      // in: float32 rows [q | k | v] (after their convolutions), SLOT_TMP: the projection's rows with the write
                        // strength's and the decay's logits and the gate; S <- g S, S += k (beta (v - S^T k))^T, o = S^T q per head over
                        // each request's rows and its state slot; out = rmsnorm(o) * vec * act(gate)
};

enum RunnerAct { RUNNER_ACT_NONE = 0, RUNNER_ACT_SILU = 1, RUNNER_ACT_GELU_TANH = 2, RUNNER_ACT_SIGMOID = 3, RUNNER_ACT_RELU = 4,
                 RUNNER_ACT_GELU_ERF = 5,       // the exact gelu, 0.5 z (1 + erf(z / sqrt 2))
                 RUNNER_ACT_SWISH_CLAMP = 6,    // EXPERTS: g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)
                 RUNNER_ACT_TANH = 7 };

struct RunnerOp {
    int kind;
    int in_slot, out_slot;
    int wanted_rows;            // 1: the operation works on the step's wanted rows only (final norm, output product)
    int n, k;                   // products: output features (GATE_UP: the width after the activation), input features
    int heads, kv_heads, head_dim, window, interleaved, writes_cache;
    int cache_group;            // which of the step's block tables indexes the pages
    int list_short, list_tiles; // ATTENTION: which of the step's lists hold its short rows and its tiles
    int w_dtype;                // EMBED: JK_F32 or JK_BF16 table
    int max_positions;          // ATTENTION: the longest context (bounds the keys of a row)
    float eps, scale, softmax_scale;    // NORM: eps, scale = the output's factor; RESIDUAL, EMBED: scale
    const void *w;              // the matrix [n (2n for GATE_UP), k] in the compute type; EMBED: the table
    const float *vec;           // NORM: the weight; QKV, LINEAR: the bias or null
    const float *cos_table, *sin_table;     // [positions, head_dim / 2] or null
    void *k_pages, *v_pages;    // [pages, kv_heads, page_size, head_dim] in the compute type
    int num_pages;
    // ---- what the mixers of csrc/mixers.cu add; all zero in the records of the plain decoder ----------------------
    int v_head_dim;             // ATTENTION, CONV_QKV, LINEAR_ATTENTION: size of a value head (0: head_dim)
    int sink;                   // ATTENTION: 1 adds a key of score 0 that has no value to every row's softmax
    int gated;                  // ATTENTION: 1 multiplies head h's output by sigmoid(SLOT_TMP[t, g_off + h])
    int act;                    // GATE_UP: RunnerAct of the gate (0 stands for silu); LINEAR_ATTENTION: of q, k and v
    int gate_act;               // LINEAR_ATTENTION: RunnerAct of the output gate
    int ld;                     // width of the fused projection's float32 rows that the record reads
    int q_off, k_off, v_off, g_off, r_off;      // columns of queries, keys, values, gate and decay projection in those rows
    int taps;                   // CONV_QKV: taps of the convolution (0: none)
    int rot_dims;               // CONV_QKV: leading elements of each head that are rotated, in pairs (2i, 2i+1)
    int per_head_norm;          // LINEAR_ATTENTION: 1 norms each head over its values (weight [dv]); 0 all heads at once
    int rank;                   // LINEAR_ATTENTION: width of the decay's projection (0: a constant per head)
    int has_kv;                 // CONV_QKV: 1 makes keys and values too (0: queries only, the cache is another layer's)
    int list_aux;               // LINEAR_ATTENTION: with list_short (requests run in one go) and list_tiles (pieces), the
                                // step's list of the requests that have pieces
    float tau, q_scale;         // LINEAR_ATTENTION: decay = sigmoid(z)^(1/tau); factor of q
    const float *conv_q, *conv_k, *conv_v;      // CONV_QKV: [channels, taps]
    const float *norm_q, *norm_k;               // CONV_QKV: weights of the whole-projection RMS norms
    const float *freq;          // CONV_QKV: [rot_dims / 2] angle per position of each pair
    const float *decay;         // LINEAR_ATTENTION: [heads] constant decays, or null
    const void *w2;             // LINEAR_ATTENTION: [heads * head_dim, rank] in the compute type, or null
    const float *b2;            // LINEAR_ATTENTION: [heads * head_dim]
    const float *bias;          // LAYERNORM: the bias
    float *state;               // CONV_QKV: tails [slots, taps - 1, channels]; LINEAR_ATTENTION: [slots, heads, dk, dv]
    // ---- what the records of csrc/blocks.cu add; read by those records only ------------------------------------------
    int in2_slot, out2_slot;    // a second input / output (LATENT_QKV, CAUSAL_CONV, SELECTIVE_SCAN)
    int rot_width;              // LATENT_QKV, LATENT_ATTENTION: elements of a head (and of a cached row) behind the plain ones
    int experts, top, ff;       // EXPERTS: how many there are, how many a row takes, their inner width
    int add;                    // EXPERTS: 1 adds to what SLOT_DELTA holds (a shared expert's output), 0 overwrites
    int out_hs;                 // HEAD_LINEAR: elements between two heads of an output row
    float eps2;                 // NORM_ADD: eps of the second norm
    float rot_mag;              // LATENT_QKV: factor of cos and sin
    float cap;                  // SOFTCAP
    const float *vec2;          // NORM_ADD: the next sublayer's norm weight
    const void *w3;             // EXPERTS: the experts' down matrices [experts, hidden, ff] (w: [experts, 2 ff, hidden])
    // NORM_ADD: vec = the norm's weight.  REINJECT: vec = the row added to every row.  LATENT_QKV: heads, head_dim (plain
    // part), rank (latent size), rot_dims, freq, norm_k (the latent norm's weight), eps, q_off, k_off (the latent's column).
    // CAUSAL_CONV: conv_q = taps [n, taps], bias, act, state = tails [slots, taps - 1, n].  SELECTIVE_SCAN: n channels, k
    // states, w2 = the step size's projection [n, rank] (compute type), b2 its bias, decay = A [n, k], vec = D, state [slots, n, k].
    // EXPERTS: n = hidden, vec = the router [experts, hidden] (float32), act = the experts' activation.
    // ---- what a window attention with kept first keys, a token-shifted recurrence and softmax-routed experts add ------------
    int keep_first;             // ATTENTION: keys at positions below this stay visible when the window has passed them
    int rot_half;               // CONV_QKV: 1 pairs element i of a head with element i + rot_dims / 2 (0: 2i with 2i + 1); rot_mag is the
                                // factor of cos and sin (0 stands for 1)
    int head_norm;              // CONV_QKV: 1 divides every head of q and k by its root mean square after the rotation (eps)
    int in_part;                // LINEAR: the product reads part `in_part` of its input slot, [parts, rows, k]
    int out_off;                // LINEAR with ld > 0: the product writes columns out_off .. out_off + n of float32 rows `ld` apart
    int decay_form;             // LINEAR_ATTENTION: the projected decay is 0: sigmoid(z)^(1/tau), 1: exp(-exp(z))
    int rank_act;               // LINEAR_ATTENTION: RunnerAct on the decay projection's `rank` columns before w2
    int score_form;             // EXPERTS: 0 sigmoid scores that multiply a unit's input; 1 softmax over all experts, the chosen ones'
                                // scores divided by their sum, multiplying the unit's output
    int into_stream;            // EXPERTS: 1 leaves SLOT_DELTA waiting to be added to the stream (by the next norm)
    float limit;                // EXPERTS: the clamp of RUNNER_ACT_SWISH_CLAMP
    // ATTENTION, CONV_QKV: `window` < 0 means chunks of -window positions: a row sees the keys of its own chunk (jk_mask_lo).
    // CONV_QKV: head_norm 2 norms every head of q and k BEFORE the rotation with the weights norm_q, norm_k [head_dim]; bias
    // [ld] is added to the projection's columns.  LATENT_ATTENTION: window.  GATE_UP: act RUNNER_ACT_SWISH_CLAMP with limit.
    // ---- what learned positions, queries through a latent, the delta rule and a gated shared expert add ------------------------
    int fixed_row;              // ADD_ROWS: the table's row that every row gets; < 0: row positions[t]
    int groups;                 // DELTA_RULE: heads of q and k (query head h reads group h / (heads / groups))
    int b_off, a_off;           // DELTA_RULE: columns of the write strength's and the decay's logits in SLOT_TMP's rows
    int q_rank;                 // LATENT_QKV: > 0: the queries pass a latent vector of q_rank elements at q_off, RMS-normed with norm_q
                                // into out2 [T, q_rank]; the heads' queries are products of it (no per-head parts are split here)
    float unit_eps;             // DELTA_RULE: q and k become x / sqrt(sum(x^2) + unit_eps)
    const float *a_log, *dt_bias;       // DELTA_RULE: [heads]; g = exp(-exp(a_log) softplus(logit + dt_bias))
    const float *router_bias;   // EXPERTS: [experts] added to the router's logits, or null
    const float *gate_w;        // EXPERTS: [n] or null: what waits in SLOT_DELTA (add = 1) is multiplied by sigmoid(gate_w . in) per row
    const float *bonus;         // LINEAR_ATTENTION: [heads, head_dim]; a row then reads the state before its own decay, its own key
                                // times the bonus: o = (S + diag(bonus) k v^T)^T q, then S = diag(a) S + k v^T
    // ATTENTION: cap > 0 caps the scores, s <- cap tanh(s / cap).
};

// What does not change from step to step and is no part's business.
struct RunnerEnv {
    int dtype;                  // JK_F32: every product on the CUDA cores in float32; JK_BF16
    int page_size, max_blocks;  // of every cache group
    int fused_norms;            // 1: steps of at most 16 rows run without norm kernels where the small-row kernels allow
    int plain_attention;        // 1: bfloat16 attention through the row kernel too
    int legacy_tensor_cores;    // 1: prefill attention on mma.sync even where tcgen05 is built
    jk::Routing routing;
    int *status;                // the word in which kernels record a bounded wait that ran out
};

// One step's batch (device arrays of the step's metadata buffer).
struct RunnerStep {
    int ntok, nreq, n_want;
    int context;                // the context length the step is planned for (the bucket of the live lengths)
    const int *tokens, *positions, *row_req, *req_start, *req_pos, *want_rows;
    const int *slot_ids;        // [nreq] the state slot of each request
    const int *block_tables[jk::MAX_CACHE_GROUPS];
    const int *lists[jk::MAX_STEP_LISTS];     // work lists that mixers asked for; null with n == ntok means "rows 0..ntok-1"
    int list_n[jk::MAX_STEP_LISTS];
};

struct RunnerBuffers {
    void *slot[RUNNER_SLOTS];
    long long bytes[RUNNER_SLOTS];
    void *workspace;                // for the library
    long long workspace_bytes;
    unsigned long long *sumsq;      // [sumsq_rows, 16] fixed-point sums of squares, one row per record
    int sumsq_rows;
};

extern "C" {
int jk_runner_bind(const RunnerFns *fns);
// Runs records [first, first + count) of `ops`.  A product that adds into the stream may wait in SLOT_DELTA for the next
// norm to add it; with `flush` one that still waits when the records end is added before the call returns (for a caller
// that goes on with code of its own), without it the wait ends with the call (nobody reads the stream after a model's
// last record).
int jk_runner_run(const RunnerEnv *, const RunnerOp *ops, int first, int count, const RunnerStep *, const RunnerBuffers *,
                  int flush, cudaStream_t);
int jk_runner_slot_bytes(const RunnerEnv *, const RunnerOp *ops, int count, int max_rows, int max_want, long long *bytes);
int jk_runner_needs_gemm_tcgen05(const RunnerEnv *, const RunnerOp *ops, int count, int max_rows);
const RunnerFns *jk_runner_fns();      // the bound table (null before jk_runner_bind)
int jk_runner_launches();
// Emitters: the records of this architecture's standard parts, written once for the Python parts and the C interface.
// Each writes its records at `out` and returns their number.
int jk_emit_attention(RunnerOp *out, const void *w_qkv, const float *b_qkv, const void *w_o, int hidden, int heads, int kv_heads,
                      int head_dim, int window, float softmax_scale, float residual_scale, const float *cos_table,
                      const float *sin_table, int interleaved, int max_positions, void *k_pages, void *v_pages, int num_pages,
                      int cache_group, int writes_cache, int list_short, int list_tiles);
int jk_emit_swiglu(RunnerOp *out, const void *w_gate_up, const void *w_down, int hidden, int intermediate, float residual_scale);
int jk_emit_rmsnorm(RunnerOp *out, const float *weight, int size, float eps, float out_scale, int wanted_rows);
int jk_emit_embedding(RunnerOp *out, const void *table, int dtype, int hidden, float scale);
int jk_emit_output(RunnerOp *out, const void *w, int vocab, int hidden);
}
