// The kernels as the host side calls them: argument checks, the choice among kernels that serve
// the same operation, then one launch.
//
// Every function works on device views, launches on the given stream (so a launch can be captured
// in a CUDA graph) and returns nothing; outputs are written into tensors the caller passes.  Sizes
// a kernel does not take are refused with UnsupportedShape before anything runs.  There is no other
// implementation behind these functions: if a kernel library cannot be loaded, the call throws.
#pragma once

#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../csrc/matrix_state.h"
#include "cache.h"
#include "device.h"

namespace sandy {
namespace ops {

enum class Act : int { None = 0, GeluNew = 1, Gelu = 2, ReluSquared = 3 };
Act act_from_name(const std::string& name);          // "gelu_new" / "gelu_tanh" / "gelu" / "gelu_erf" / "relu_squared" / "none"

// Where the launches of one step go and where kernels report trouble.
struct Launch {
    cudaStream_t stream = nullptr;
    int* status = nullptr;             // device int: bit 0 bad token id or NaN logits, bit 1 bad position
    int* kernel_status = nullptr;      // device int: expired waits, pages that do not exist (see kernel_status_text)
};
const char* kernel_status_text();

// Device time per kernel class, behind a switch (the reference times every op the same way through
// EngineRunOptions::profileKernel, src/engine/Engine.h:56-60, src/engine/Engine.cpp:887-921).  While
// it is on, every launch outside a graph capture gets a pair of CUDA events; `profile_report` waits
// for them and returns per class the launches, microseconds, bytes that had to move and operations.
struct ProfileRow {
    std::string op_class;
    long long calls = 0;
    double us = 0, bytes = 0, flops = 0;
};
void profile_enable(bool on);
// Families of launches that are skipped from now on ("layernorm", "attention", "kv_append", "product",
// "product <N>x<K>"): for timing what a family costs inside a step; results are garbage meanwhile.
void leave_out(const std::vector<std::string>& families);
void force_tile(int64_t N, int64_t K, int tile);      // tcgen05 variant for products of W [N, K]; 0: the tuner's
std::vector<ProfileRow> profile_report();              // also clears what was gathered

int sm_count();                                        // streaming multiprocessors of the current device
void spin(cudaStream_t stream, long long nanoseconds); // keeps the stream busy (timing loops queue launches behind it)

void embed_positions(const Launch& l, const int* ids, const int* positions, const Tensor& wte, const Tensor* wpe,
                     Tensor& out, int n_tokens);
void layernorm(const Launch& l, const Tensor& x, const Tensor& gamma, const Tensor* beta, float eps, Tensor& out,
               const int* rows, int n_rows);

// Where the key/value columns of a fused q/k/v product belong: the layer's cache view and the
// step's index arrays.  `written` is set by the product if its kernel did the write.
struct KVTarget {
    KVView cache;
    const int* block_table = nullptr;
    int max_blocks = 0;
    const int* token_seq = nullptr;
    const int* positions = nullptr;
    int q_cols = 0, kv_cols = 0;
    bool written = false;
};

// A LayerNorm that the product's kernel runs itself on the float32 rows `x` (decode steps).
struct FusedNorm {
    Tensor x;
    Tensor gamma;
    const Tensor* beta = nullptr;
    float eps = 0.0f;
};

// out = act(a @ W + bias) + residual.  W is [K, N], or [N, K] with w_out_in.
void gemm_simt(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, bool w_out_in, Act act,
               const Tensor* residual);
// tcgen05 tensor cores: a bfloat16 [M, K], w bfloat16 [N, K].  tile_n 0 lets the tuner (256 rows and more) or the
// kernel choose; see GEMM_VARIANTS in ops.cpp for the codes.
bool tensor_core_gemm_supported(int64_t K, int64_t N);
void gemm_tc(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
             const Tensor* residual, int tile_n = 0, KVTarget* kv = nullptr);
// Weight streaming for up to 64 rows (a decode step); optional LayerNorm prologue and key/value write.
bool skinny_norm_fusable(const FusedNorm& n, int64_t K, DType out_dtype);
// Up to how many rows running the norm inside the product pays.  Every block of the product norms all
// rows itself, so that traffic grows with rows x blocks, while the norm as a launch of its own costs a
// fixed 1.5 us or so behind programmatic dependent launch.  Whole decode steps of GPT-2 small (ms, norm
// inside / norm apart): 1 request .244 / .250, 2: .255 / .262, 4: .267 / .270, 6: .290 / .285, 7: .297 /
// .288, 8: .303 / .294, 12: .381 / .341, 16: .409 / .361.
constexpr int kSkinnyNormPaysRows = 4;
// ... and up to which K: the blocks' norms also grow with the row's width.  One request, ms a decode step, norm
// inside / apart: GPT-2 small (K 768) .244 / .250, medium (1,024) .572 / .573, xl (1,600) 3.45 / 2.80.
constexpr int kSkinnyNormPaysK = 1024;
void gemm_skinny(const Launch& l, const Tensor* a, const FusedNorm* norm, const Tensor& w, const Tensor* bias, Tensor& out,
                 Act act, const Tensor* residual, KVTarget* kv = nullptr);
constexpr int kSkinnyMaxRows = 64;
// tcgen05 with the weight as the wide operand and K split over a cluster, for 17 to 64 rows (gemm_small.cu).
// small_gemm_kernel: which kernel a bfloat16 product of 17 to 64 rows gets, from its shape alone.
// The split-K kernel also takes 65 to 256 rows (a short prompt step, or a portion of one): products with a
// long K and few row tiles, which the tile kernels run on a handful of CTAs (128 x 768 x 3072: six CTAs of 48
// k-steps each, 18 us inside the step).
// Prompt steps of one request, us, tile kernels / split-K for the down-projection: 65 tokens 642 / 556, 128: 686 /
// 595, 129: 680 / 640, 192: 673 / 683, 256: 692 / 697: it pays up to 128 rows (one 128-wide side); the kernel
// itself takes up to 256.
constexpr int kSmallMaxRows = 256;
constexpr int kSmallPaysRows = 128;
constexpr int kSmallManyRowsMinK = 2048;
enum class SmallGemm { Skinny, SplitK };
SmallGemm small_gemm_kernel(int64_t M, int64_t N, int64_t K);
void gemm_small(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
                const Tensor* residual, KVTarget* kv = nullptr);

void kv_append(const Launch& l, const Tensor& k_src, const Tensor& v_src, const KVView& cache, const int* block_table,
               int max_blocks, const int* token_seq, const int* positions);

// What an attention launch needs to know about the step.
struct AttentionStep {
    int n_tokens = 0, n_seqs = 0, max_q_len = 0;
    const int* token_seq = nullptr;
    const int* positions = nullptr;
    const int* q_start = nullptr;
    const int* kv_before = nullptr;
    const int* block_table = nullptr;
    int max_blocks = 0;
    // from the step's host-side lists, for the profile's figures only: keys the step's requests hold
    // after it, and (query, key) pairs the causal attention looks at
    double kv_tokens = 0, pairs = 0;
};
// What some attention layers add to the softmax: a sink per head (float32 [H]: exp(sink) joins the denominator and
// nothing else) and a factor on each head's output (float32 [T, H], e.g. a sigmoid gate).  Either may be null.
// Two rules on the scores: `softcap` > 0 presses a score into softcap * tanh(score / softcap) before the softmax;
// `chunk` > 0 lets a query at position pos see only the keys of its own chunk, j >= pos - pos % chunk (chunks are counted
// from position 0 of the request).  Kernels without a form for a rule leave such steps to those that have one.
struct AttentionExtras {
    const float* sink = nullptr;
    const float* out_gate = nullptr;
    float softcap = 0.0f;
    int chunk = 0;
    // A learned bias by distance: entry min(i - j, n_dist - 1) of the head's row of dist_bias (float32 [H, n_dist]) joins
    // the score of query i and key j after the scale and the cap.  Null: none.
    const float* dist_bias = nullptr;
    int n_dist = 0;
};
// The widest head any attention kernel takes (the general kernel; the tensor-core prompt kernels take up to 128, the
// decode kernels 16 / 32 / 64 / 128 and, in bfloat16, 256).
constexpr int kMaxHeadDim = 640;
// From this many query heads per key/value head on, a decode step's attention takes sixteen heads of a group as the
// rows of one tensor-core product (attention_decode_shared.cu, bfloat16, heads up to 128).
constexpr int kSharedKvMinHeads = 4;
constexpr int64_t kSharedKvMinTriples = 40000;      // tokens x heads x keys (the block table's width) from which it pays
// Attention of a step's tokens over the cache: picks the kernel for the step's shape.
void attention(const Launch& l, const AttentionStep& s, const Tensor& q, const KVView& cache, Tensor& out, int n_heads,
               float scale, int window, Workspace& ws, const AttentionExtras* extras = nullptr);
int decode_splits(int n_tokens, int n_heads, int max_kv, int sms = 0);

// ---- RMS norms and what goes with them (rmsnorm.cu, elementwise.cu) ------------------------------------------
struct StepSeqs {                                                  // the step's requests, as kernels with a state per request need them
    int n_tokens = 0, n_seqs = 0;
    const int* token_seq = nullptr;
    const int* q_start = nullptr;
    const int* seq_slots = nullptr;
};
// out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * gain; x float32, gain float32 [width] or null.
void rmsnorm(const Launch& l, const Tensor& x, const Tensor* gain, float eps, Tensor& out, const int* rows, int n_rows);
// Token shift behind the norm: h[t] = norm(x[t]) * gain, out[t] = h[t] + (h[t-1] - h[t]) * mix, where the h before a
// request's first token of the step is the first x.cols floats of its state row (zeros at a request's very first
// token: a slot is cleared on admission), and the row then takes the h of the request's last token.  All 32-bit; out
// in its own type.  `max_q_len` is the step's longest portion (one launch when it is 1, two otherwise).
void rmsnorm_shift(const Launch& l, const StepSeqs& s, const Tensor& x, const Tensor* gain, float eps, const Tensor& mix,
                   const StateView& state, Tensor& out, int max_q_len);
// x += mult * y / sqrt(mean(y^2) + eps) * gain; both float32.
void rmsnorm_add(const Launch& l, const Tensor& y, const Tensor* gain, float eps, float mult, Tensor& x);
enum class GateAct : int { Sigmoid = 0, Silu = 1 };
// Per (token, head): out = o / sqrt(mean over the head (o^2) + eps) * gain * act(gate) * scale.  o float32 [T, H * dim];
// gain float32, [dim] shared by the heads or [H * dim]; gate [T, H * dim] or null.
void head_norm_gate(const Launch& l, const Tensor& o, const Tensor* gain, const Tensor* gate, GateAct act, float scale,
                    float eps, int n_heads, Tensor& out);
enum class GluAct : int { Silu = 0, GeluTanh = 1 };
// out = act(a) * b, element by element (a and b may be column ranges of one matrix).
void glu(const Launch& l, const Tensor& a, const Tensor& b, GluAct act, Tensor& out);
// out = g * sigmoid(alpha * g) * (u + 1) with g = min(a, limit), u = clamp(b, -limit, limit), element by element.
void glu_clamped(const Launch& l, const Tensor& a, const Tensor& b, float limit, float alpha, Tensor& out);
// out = x rounded to out's type (out may be a column range of a wider matrix); x float32.
void cast_cols(const Launch& l, const Tensor& x, Tensor& out);

// x += gain * y (+ gain2 * y2): sublayer results joining the stream through a factor per channel; all float32.
void scale_add(const Launch& l, const Tensor& y, const Tensor& gain, const Tensor* y2, const Tensor* gain2, Tensor& x);
// x *= s, float32 (logits times a constant).
void scale(const Launch& l, Tensor& x, float s);
// x += x0 + row: x and x0 float32 [T, width], row float32 [width]; x0 and row may each be null.
void stream_add(const Launch& l, Tensor& x, const Tensor* x0, const Tensor* row);
// x = cap * tanh(x / cap), float32 (logits pressed into (-cap, cap)).
void softcap(const Launch& l, Tensor& x, float cap);

// ---- attention over a latent (latent_prepare.cu, grouped_gemm.cu) ---------------------------------------------
// What the cache of such a layer holds per token, [latent | shared rotated key part | zeros], is key and value at
// once (a one-plane page), and every query head becomes [U_k^T q | rotated part | zeros] of the same width.
struct LatentPrepare {
    int q_rank = 0;                    // > 0: queries pass a latent of their own; its norm is written to q_latent
    int kv_rank = 0, rot_dim = 0;      // columns of `down`: q_rank, then kv_rank, then rot_dim
    const float* q_gain = nullptr;     // float32 [q_rank]
    const float* kv_gain = nullptr;    // float32 [kv_rank]
    float eps = 0.0f;
    const float* freq = nullptr;       // float32 [rot_dims / 2]; neighbours (2i, 2i+1) are a pair
    int rot_dims = 0;                  // how many of the rot_dim entries turn
    int n_heads = 0, qk_dim = 0;       // q is [T, n_heads * (qk_dim + rot_dim)]
    bool write_cache = true;
};
// down float32 [T, q_rank + kv_rank + rot_dim]; q (read where rot_dim > 0) and q_abs [T, n_heads * cache.head_dim] of the
// cache's dtype; q_latent [T, q_rank] of the cache's dtype or null.
void latent_prepare(const Launch& l, const LatentPrepare& p, const Tensor& down, const Tensor* q, const KVView& cache,
                    const int* block_table, int max_blocks, const int* token_seq, const int* positions, Tensor* q_latent,
                    Tensor& q_abs);
// out[t, g * o_gcols + n] = sum_k w[g][n][k] * a[t, g * a_gcols + k]: one small matrix per head.  w is [G * N, K].
void head_product(const Launch& l, const Tensor& a, int a_gcols, const Tensor& w, int n_groups, Tensor& out, int o_gcols);

// ---- mixture of experts (moe.cu, grouped_gemm.cu) ---------------------------------------------------------------
// The routing of a step, all device data: entry t * top + j is the j-th choice of token t.
struct Routing {
    int n_tokens = 0, n_experts = 0, top = 0;
    int* expert_of = nullptr;          // [n_tokens * top]
    float* weight_of = nullptr;        // [n_tokens * top], softmax over a token's chosen logits
    int* group_start = nullptr;        // [n_experts + 1] slots of every expert
    int* entry_of_slot = nullptr;      // [n_tokens * top]
    int* slot_of_entry = nullptr;      // [n_tokens * top]
};
// logits float32 [T, E] (+ bias float32 [E] or null) -> the routing's arrays.
void moe_route(const Launch& l, const Tensor& logits, const Tensor* bias, const Routing& r);
// Routing by scores: s = sigmoid(logit); the choice is by s + correction among the experts of the `keep_groups` best of
// `n_groups` equal groups of neighbours (a group's score: the sum of its `group_rank` largest choice scores); the weights
// are the chosen s over their sum (+ norm_eps), times weight_scale.
struct ScoredRoute {
    int n_groups = 1, keep_groups = 1, group_rank = 2;
    float weight_scale = 1.0f, norm_eps = 0.0f;
};
void moe_route_scored(const Launch& l, const Tensor& logits, const Tensor* correction, const ScoredRoute& rule, const Routing& r);
// Routing by softmax scores: s = softmax over all experts' logits; the choice is by s + correction; the weights are the
// chosen s themselves times weight_scale, over their sum (+ norm_eps) only with `renormalize`.
struct SoftmaxRoute {
    float weight_scale = 1.0f, norm_eps = 0.0f;
    bool renormalize = false;
};
void moe_route_softmax(const Launch& l, const Tensor& logits, const Tensor* correction, const SoftmaxRoute& rule, const Routing& r);
enum class ExpertAct : int { None = 0, ReluSquared = 1 };
// out[s] = act(W_e a[row(s)]) for the slots s of every expert e; w [E * N, K]; with `gather` a slot reads its token's
// row of `a` ([T, K]), else row s ([T * top, K]).  out [T * top, N].
// bfloat16 products whose rows start on 16-byte boundaries run on tcgen05 (grouped_gemm_tc.cu), which wants an
// expert's rows one after another: with `gather` the rows are first copied into `sorted` ([T * top, K] of a's type;
// without that scratch the product stays on the mma.sync tiles).  float32 and odd sizes take grouped_gemm.cu.
// The tcgen05 kernel is ahead at every step size, the copy included (width 1,536, 16 experts of 2,048, 2 a token; us
// for the up- and the down-projection, mma.sync tiles / tcgen05): 8,192 tokens 379 + 374 / 117 + 137; 2,048: 124 +
// 120 / 44 + 50; 64: 38 + 42 / 21 + 22; 8: 31 + 32 / 28 + 35; 1: 22 + 24 / 13 + 14; the copy 5 to 18.  Whole decode
// steps of 4 layers, ms, 1 / 8 requests: 0.326 / 0.457 on the mma.sync tiles, 0.272 / 0.434 on tcgen05.
void expert_product(const Launch& l, const Routing& r, const Tensor& a, bool gather, const Tensor& w, ExpertAct act, Tensor& out,
                    Tensor* sorted = nullptr);
// y[t] (+)= sum_j weight[t, j] * rows[slot of (t, j)]; rows float32 [T * top, width], y float32 [T, width].
void moe_combine(const Launch& l, const Routing& r, const Tensor& rows, Tensor& y, bool add);
// The same where the experts from n_real on have no matrices and hand their input on: such an entry contributes
// weight * h[t] (h [T, width], the feed-forward's input) instead of a computed row.
void moe_combine_identity(const Launch& l, const Routing& r, int n_real, const Tensor& h, const Tensor& rows, Tensor& y, bool add);

// ---- between a q/k/v projection and attention (attention_prepare.cu) -----------------------------------------
struct AttentionPrepare {
    int n_heads = 0, n_kv_heads = 0, qk_dim = 0, v_dim = 0;       // the cache's head size is cache.head_dim >= both
    int q_off = 0, k_off = 0, v_off = 0;                           // first columns of q, k, v in the projection
    const float* q_gain = nullptr;                                 // RMS norm over the whole q row / k row, or null
    const float* k_gain = nullptr;
    float eps = 0.0f;
    const float* freq = nullptr;                                   // rotary frequencies [rot_dims / 2], or null
    int rot_dims = 0;
    const float* gate_in = nullptr;                                // float32 [T, ld_gate]: per-head gate pre-activations
    int ld_gate = 0;
    float* gate_out = nullptr;                                     // float32 [T, H]: sigmoid(gate_in) * gate_scale
    float gate_scale = 1.0f;
    const float* q_head_scale = nullptr;                           // float32 [H]: a factor on each query head, or null
    float v_unit_eps = 0.0f;                                       // > 0: every value head over its root mean square (this eps)
    bool per_head_norm = false;                                    // every query and key head over its own root mean square (eps);
                                                                   // the gains may then be null
    float q_pos_coef = 0.0f;                                       // with q_pos_every > 0 the query at position p is multiplied by
    int q_pos_every = 0;                                           // 1 + q_pos_coef * ln(floor((p + 1) / q_pos_every) + 1)
    bool write_cache = true;
};
void attention_prepare(const Launch& l, const AttentionPrepare& p, const Tensor& proj, const KVView& cache,
                       const int* block_table, int max_blocks, const int* token_seq, const int* positions, Tensor& q_out);

// ---- recurrent mixers with a matrix state per head (matrix_state.cu) -------------------------------------------
// Columns of a head's state that one thread block owns; the matrix memory keeps n and m once per such block.
constexpr int kMatrixStateCols = SANDY_MATRIX_STATE_COLS;
int64_t mlstm_state_floats(int n_heads, int qk_dim, int v_dim);
struct DeltaShape { int n_heads = 0, n_qk_heads = 0, qk_dim = 0, v_dim = 0, n_taps = 0; };
// conv + silu + unit vectors + gates.  proj [T, >= channels] (q, k, v channels first); taps float32 [channels, n_taps];
// gates float32 [T, 2H] (beta's pre-activation, then the decay's); qkv float32 [T, channels]; bg float32 [T, 2H]
// (beta, then the logarithm of the decay).
void delta_prepare(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& proj, const Tensor& taps,
                   const Tensor& gates, const float* a_log, const float* dt_bias, const StateView& state, int64_t tail_off,
                   float q_scale, Tensor& qkv, Tensor& bg);
void conv_tail(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& proj, const StateView& state,
               int64_t tail_off);
// From how many tokens of one request on a step's recurrence runs a chunk of tokens at a time (parallel inside the
// chunk) instead of token by token.  Token by token costs about 0.8 us a token and head (a dependent chain of some 240
// instructions), a chunk of 32 about 2 us, so the chunked kernel is ahead from a handful of tokens on.
constexpr int kChunkedFrom = 8;
// `max_q_len`: the step's longest portion.  Below kChunkedFrom only the token-by-token kernel is launched; from there
// on both are, each taking the requests of its own kind (which requests those are is read on the device).
void delta_scan(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& qkv, const Tensor& bg,
                const StateView& state, Tensor& out, int max_q_len);
struct MlstmShape { int n_heads = 0, qk_dim = 0, v_dim = 0, q_off = 0, k_off = 0, v_off = 0; float cap = 1.0f, q_scale = 1.0f; };
// gates float32 [T, >= 2H]: input-gate pre-activations, then forget-gate ones; gate_bias float32 [2H].
void mlstm_scan(const Launch& l, const StepSeqs& s, const MlstmShape& m, const Tensor& proj, const Tensor& gates,
                const float* gate_bias, const StateView& state, Tensor& out, int max_q_len);

// The last n_taps - 1 rows of `rows` ([T, channels], any pitch) of every request into its state at tail_off, as the
// convolutions above keep theirs (rows before the step come from the old tail).
void conv_tail(const Launch& l, const StepSeqs& s, const Tensor& rows, int n_taps, const StateView& state, int64_t tail_off);

// ---- a selective state-space mixer with one decay per head (ssm_state.cu) ----------------------------------------
struct SsmShape { int n_heads = 0, n_groups = 0, state = 0, v_dim = 0, n_taps = 0; };
int64_t ssm_state_floats(const SsmShape& m);                       // S [H][P][N]; the convolution's tail follows it
// proj: the x, B and C channels ([T, H * P + 2 G * N], a column range of the input projection); taps float32 [channels,
// n_taps], conv_bias float32 [channels] or null; dt_raw float32 [T, H]; xbc float32 [T, channels] = silu(conv + bias);
// dta float32 [T, 2H]: dt = softplus(raw + dt_bias), then -exp(a_log) dt.  The convolution's tail in the state moves on by
// the step's tokens: in the same launch when the step's longest portion `max_q_len` is one token, by conv_tail otherwise.
void ssm_prepare(const Launch& l, const StepSeqs& s, const SsmShape& m, const Tensor& proj, const Tensor& taps, const Tensor* conv_bias,
                 const Tensor& dt_raw, const float* dt_bias, const float* a_log, const StateView& state, int64_t tail_off,
                 Tensor& xbc, Tensor& dta, int max_q_len);
// S <- exp(dta[1]) S + dt B x^T; out = S^T C + d_skip x, float32 [T, H * P]; d_skip float32 [H] or null.
void ssm_scan(const Launch& l, const StepSeqs& s, const SsmShape& m, const Tensor& xbc, const Tensor& dta, const float* d_skip,
              const StateView& state, Tensor& out);
// out = (y * silu(z)) over its root mean square in `groups` equal parts of a row (eps inside the root), times gain.
void gated_group_norm(const Launch& l, const Tensor& y, const Tensor& z, const Tensor* gain, float eps, int groups, Tensor& out);

// ---- a residual stream in several copies (streams.cu) -------------------------------------------------------------
// What one pass over the streams X (float32 [T, S * width]) does, each part optional and in this order:
//   write   X_t <- sum_s mix[s, t] X_s + out_w[t] * y * sigmoid(gate + gate_bias)     (y, gate float32 [T, width])
//   sum     sum_out = sum_s X_s                                                        (float32 [T, width])
//   read    h = LayerNorm(sum_s in_w[s] X_s) * gain, no offset                         (h [T, width] of the compute type)
struct StreamsStep {
    const Tensor* y = nullptr;
    const Tensor* gate = nullptr;
    const Tensor* gate_bias = nullptr;       // float32 [width]
    const Tensor* mix = nullptr;             // float32 [S, S], indexed [from, to]
    const Tensor* out_w = nullptr;           // float32 [S]
    const Tensor* in_w = nullptr;            // float32 [S]
    const Tensor* gain = nullptr;            // float32 [width]
    float eps = 0.0f;
    Tensor* h = nullptr;
    Tensor* sum_out = nullptr;
    // With the read, in a step in which EVERY request brings one token: the short convolution of canon_conv in the same
    // launch, conv_out = h + conv(h), and the request's tail moved on by the token (canon_conv + conv_tail otherwise).
    const Tensor* taps = nullptr;            // float32 [width, n_taps]
    int n_taps = 0;
    const StateView* state = nullptr;
    int64_t tail_off = 0;
    const StepSeqs* seqs = nullptr;
    Tensor* conv_out = nullptr;
};
int streams_max();
void streams_step(const Launch& l, Tensor& X, int n_streams, const StreamsStep& step);
void streams_spread(const Launch& l, const Tensor& x, Tensor& X, int n_streams);
// c = h + conv(h): a short causal convolution over time on every channel (taps float32 [width, n_taps], the last column
// the token's own), rows before the step from the request's tail at tail_off of its state.
void canon_conv(const Launch& l, const StepSeqs& s, const Tensor& h, const Tensor& taps, int n_taps, const StateView& state,
                int64_t tail_off, Tensor& c);
// x[t] = wte[id] + bigram[(id_before * mul_prev + id * mul_cur) mod buckets] + wpe[pos]; a request's first token reads
// row `buckets`; the token before a step's first one is the int32 state of the request, which then takes the step's last.
struct BigramEmbed { int buckets = 0; long long mul_prev = 0, mul_cur = 0; };
void embed_bigram(const Launch& l, const StepSeqs& s, const int* ids, const int* positions, const Tensor& wte, const Tensor& bigram,
                  const Tensor* wpe, const BigramEmbed& b, const StateView& state, Tensor& x, int max_q_len);

// Choose one token per row of float32 `logits`; per-row option arrays may be null.  With `feedback`
// the drawn token also replaces the row's input token, its position moves on, and the token is
// recorded in burst_tokens[row_step[r], r]; `uniform` then holds [steps, rows] numbers.
struct SampleFeedback {
    int* token_ids = nullptr;
    const int* logit_rows = nullptr;
    int* positions = nullptr;
    int* burst_tokens = nullptr;
    int* row_step = nullptr;
};
void sample(const Launch& l, const Tensor& logits, int* out_tokens, const float* temperature, const int* top_k,
            const float* top_p, const float* uniform, const SampleFeedback* feedback);

}  // namespace ops
}  // namespace sandy
