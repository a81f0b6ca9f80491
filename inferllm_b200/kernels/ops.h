// The C++ faces of the CUDA kernels: argument checks, the choice of a kernel for the sizes at
// hand, scratch and results from the step arena, the launch.
//
// Every function launches on the device's stream and returns without synchronising.  A size that a
// kernel cannot take is refused with a KernelError that names it; nothing falls back to another
// implementation, except that the plain matrix product of the bfloat16 mode is the library's
// (cuBLAS), as the reference's is (cublasSgemm, src/kern/gpu/kernel_gpu.cu:420-435).  Results are cut
// from the device's step arena and live until the next step rewinds it.
#pragma once
#include <cstdint>
#include <string>

#include "cache/cache.h"
#include "device/device.h"

namespace illm {

// A row-major matrix on the device: rows x cols elements of `dtype`, rows contiguous.
struct Mat {
    void* p = nullptr;
    long long rows = 0, cols = 0;
    DType dtype = DType::BF16;
    // Rows that the allocation really holds (>= rows): prompt-sized bfloat16 activations are allocated
    // in whole buckets of 64 rows, so that the library's products only ever see multiples of 64 rows
    // (it chooses a kernel per shape, which costs milliseconds the first time a shape is seen).
    long long rows_held = 0;
    size_t bytes() const { return (size_t)rows * cols * dtype_size(dtype); }
};

// The K slices of a split matrix product that have not been added up yet: float32
// [splits, rows, cols].  The norm, the rotation and the decode attention kernels take it in place of
// the finished matrix and do the addition themselves (ascending order of the slice, as the
// stand-alone reduction does), which saves a kernel per product in a decode step.
struct Partials {
    float* ws = nullptr;
    int splits = 0;
    long long rows = 0, cols = 0;
};

// Either a finished matrix or unreduced slices.
struct MatOrPartials {
    Mat m;
    Partials part;
    bool is_partials() const { return part.ws != nullptr; }
    long long rows() const { return is_partials() ? part.rows : m.rows; }
    long long cols() const { return is_partials() ? part.cols : m.cols; }
};

// What every part sees of a step, on the device: int32 arrays in one buffer.
struct StepView {
    const int* ids = nullptr;         // [T] token id
    const int* token_pos = nullptr;   // [T] absolute position
    const int* token_seq = nullptr;   // [T] index of the token's sequence within the step
    const int* want_rows = nullptr;   // [K] rows (among the T tokens) whose logits are wanted
    const int* slots = nullptr;       // [B]
    const int* seq_lens = nullptr;    // [B] length after the step
    const int* cu_q = nullptr;        // [B + 1] token offsets of the sequences
    int T = 0, B = 0, K = 0;
    int max_q = 0;                    // the most tokens one sequence brings
    long long max_len = 0;            // the longest sequence after the step
    long long max_seq_len = 0;        // the longest sequence the cache allows (sizes decode grids and scratch)
    bool is_decode = false;           // one token per sequence
    int* err = nullptr;               // the step's error word
};

namespace ops {

enum class GemmBackend { Auto, TC, Library };
// Which kernel runs the bfloat16 matrix products.  TC: the package's tcgen05 kernels for every
// product they can take (K a multiple of 8): gemm_tc.cu up to 128 tokens, the SM-pair kernel
// gemm_tc2.cu above; Library: cuBLAS; Auto (default): the tcgen05 kernel for small decode batches (at
// most 16 tokens), where its swapped, split-K form with weight prefetch across kernel boundaries is
// faster than the library (74.8 against 89.5 us for the four products of a 7B layer at batch 1, 78.1
// against 79.4 at batch 16), and the library for larger ones.  From 17 to 64 tokens the kernel alone
// still matches the library (85.0 against 88.1 us at 64 tokens, back to back), but its float32 K
// slices grow with the tokens and their readers (the norms, the fused attention) pay for them: whole
// 7B decode steps at context 600 take 4.35 ms with the library and 4.47 ms with the kernel at batch
// 24, 4.77 and 5.01 at batch 32, 5.86 and 6.17 at batch 48.  Gate/up products of prompts from 512
// tokens on run on the SM-pair kernel with the activation as their epilogue.
GemmBackend gemm_backend_from_name(const std::string& name);
const char* gemm_backend_name(GemmBackend b);

constexpr int kLibraryRowBucket = 64;
constexpr int kGemmTcMaxTokensAuto = 16;
constexpr int kGatedPromptsOnTcMinTokens = 512;
constexpr int kMaxHeadDimGeneric = 256;
constexpr int kMoeTcgen05MinRows = 256;      // (token, expert) pairs from which a routed feed-forward's products run on tcgen05
constexpr int kMaxNormWidth = 200 * 1024 / 4;
constexpr int kDecodeChunk = 256, kGqaDecodeChunk = 128, kGqaDecodeMinGroup = 4, kRingDecodeMaxSplits = 32;

// An uninitialised [rows, cols] activation from the step arena; for prompt-sized bfloat16 rows the
// head of a buffer of whole buckets.
Mat new_mat(Device& dev, long long rows, long long cols, DType dtype);

// ---- policies (pure functions, tested on the CPU)

// How many slices of K a decode-sized product (M <= 64) is cut into, so that about two blocks per SM
// stream the weights; 1 for larger M.
int gemm_tc_splits(long long M, long long N, long long K, int n_sms);
// Blocks per (token, kv head) of the ring decode attention, by a small model of the kernel's time
// fitted to measurements (13B size, batch 8, context 4096, 320 pairs: 1 split 129 us, 6 splits 106 us;
// 160 pairs: 1 split 56 us, 2 splits 69 us).  Two blocks fit an SM, so 2 * n_sms run at once.  Up to
// that number the kernel streams at the memory rate once about 160 blocks are at work.  Beyond it the
// blocks run in waves, and a last wave of few blocks still takes 0.43 of a full one (a block alone is
// bound by what one SM can take in), so a grid a little larger than one wave is the worst and one of
// many waves is fine again.  Splits cost their partial results and the merge (2.5 us and 0.7 us per
// split), every wave about 1 us of start-up.  At most one split per 64-key tile and at most 32.
int attention_decode_ring_splits(long long T, int n_kv_heads, long long max_len, int head_dim, int n_sms,
                                 double stream_bytes_per_us = 6.6e6);
bool attention_decode_ring_supported(DType dtype, int nh, int nkv, int d, int page_size);
bool attention_decode_supported(DType dtype, int nh, int nkv, int d, int page_size);
bool attention_decode_gqa_supported(DType dtype, int nh, int nkv, int d);
bool attention_prefill_supported(DType dtype, int nh, int nkv, int d);
bool attention_prefill_tc_supported(DType dtype, int nh, int nkv, int d, int page_size);
// Which attention kernel a configuration gets for prompts and for single tokens (for the log line at
// engine start): "prefill_tc/decode_ring", "generic/generic", ...
std::string attention_kernels_for(DType dtype, int nh, int nkv, int d, int page_size);

// ---- kernels

Mat embedding(Device& dev, const int* ids, long long T, const Mat& table, int* err);
// table[id] * scale plus, with inv_freq (float32 [ceil(H / 2)] on the device), the sinusoid position vector
// (sin(p f_i), cos(p f_i)) in entries (2i, 2i + 1)
Mat embedding_scaled(Device& dev, const StepView& ctx, const Mat& table, float scale, const float* inv_freq);
// Layer norm (weight, no bias) around the float32 stream: resid += ln(delta) * post_w (delta, post_w nullptr: nothing
// is added), then ln(resid) * w in `out_dtype` (w nullptr: the addition alone, an empty matrix comes back).  rows
// (int32, device) gathers: only those rows are made and resid is left as it is.
Mat layernorm_sandwich(Device& dev, const Mat& resid, const Mat* delta_f32, const Mat* post_w_f32, const Mat* w_f32, float eps, DType out_dtype,
                       const int* rows, long long n_rows);
// y = act(conv(x) + bias) (+ x): a causal convolution over time per channel of columns [x_off, x_off + C) of the
// float32 rows x, `taps` taps w [C, taps] (float32, the last the token's own), the rows before the step from the
// sequence's state ([taps - 1, C] at state_off of the slot's elements), which is renewed if `update`.  Written to
// columns [o_off, o_off + C) of `out`.
struct ShortConv {
    int x_off = 0, C = 0, taps = 1;
    const float *w = nullptr, *bias = nullptr;
    int act = 0;              // 0: none, 1: silu
    bool residual = false;
    long long state_off = 0;
    bool update = true;
};
void short_conv(Device& dev, const Mat& x_f32, const ShortConv& p, const StepView& ctx, const StateView& st, const Mat& out, int o_off);
// y = rmsnorm(resid (+ delta)) * weight; resid is updated in place when write_resid.  rows (int32
// [n_rows], device) gathers: only those rows are normed and y is [n_rows, H].
Mat add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& weight, float eps, DType out_dtype,
                const int* rows, long long n_rows, bool write_resid);
void residual_add(Device& dev, const Mat& resid, const MatOrPartials& delta);
Mat materialize(Device& dev, const Partials& p, DType dtype);
Mat swiglu(Device& dev, const MatOrPartials& gu);
Mat gemm_f32(Device& dev, const Mat& x, const Mat& w);
MatOrPartials gemm_bf16_tc(Device& dev, const Mat& x, const Mat& w, DType out_dtype, int splits /* 0: by policy */, bool defer_reduce);
Mat gemm_bf16_tc2(Device& dev, const Mat& x, const Mat& w, DType out_dtype, bool gated, int act = 1 /* kActSilu */);
// x [M, K] . w [N, K]^T.  defer_reduce allows the result to come back as unreduced slices (only a
// caller that hands it to add_rmsnorm, the rotation or the fused decode attention asks).
MatOrPartials linear(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, DType out_dtype, bool defer_reduce);
// act(gate) * up of x . w^T, where w's rows 2i, 2i + 1 are the gate and the up row of output i (act: a GateAct, silu
// by default); the product kernels of the package apply it in their epilogues.
Mat linear_gated(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, int act = 1 /* kActSilu */);

struct Geometry { int n_heads, n_kv_heads, head_dim; };
// Rotate Q (and K) of the packed projection and store K, V in the cache pages.  cos_sin: float32
// [positions, rot_dim / 2, 2] or nullptr with rot_dim 0.  Returns the matrix whose first
// n_heads * head_dim columns hold the rotated queries: qkv itself (rotated in place), or, if qkv came
// as unreduced slices, a new one (the slices are added up on the way).
Mat rope_kv_write(Device& dev, const MatOrPartials& qkv, const float* cos_sin, int rot_dim, long long n_pos, const StepView& ctx,
                  const KVView& kv, Geometry g);
// Options of the generic attention kernel beyond the plain softmax attention: a per-head sink in the
// softmax denominator (float32 [n_heads]), and a per-head output gate, sigmoid(gate[t * gate_stride + h])
// (float32).  The value head size is the cache entry's (KVView::v_head_dim).
struct AttentionExtras {
    const float* sinks = nullptr;
    const float* gate = nullptr;
    int gate_stride = 0;
    // the tensor-core prompt kernel keeps sixteen bits of the softmax weights' mantissa (two bfloat16
    // terms) instead of eight; the other kernels have float32 weights anyway
    bool wide_weights = false;
};
Mat attention_generic(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                      const AttentionExtras* extras = nullptr);
Mat attention_decode(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len);
Mat attention_decode_gqa(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len);
struct FusedRope { const float* cos_sin; int rot_dim; long long n_pos; bool write_kv; int* step_err; };
Mat attention_decode_ring(Device& dev, const MatOrPartials& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                          long long max_len, int splits /* 0: by policy */, const FusedRope* rope, const AttentionExtras* extras = nullptr);
Mat attention_prefill(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);
Mat attention_prefill_tc(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                         const AttentionExtras* extras = nullptr);
// The split-key decode kernel on CUDA cores (float32 scores and weights) with sinks and gates in its merge.
Mat attention_decode_ex(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len,
                        const AttentionExtras& extras);
// Attention with extras: the tensor-core prompt kernel and the split-key decode kernel where the
// sizes allow (bfloat16, keys and values of one size, 64 or 128), the general kernel otherwise.
Mat attention_ex(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const AttentionExtras& extras);
// Attention whose heads' scores are mixed before the softmax (mix float32 [n_heads, n_heads] or nullptr), with a
// logarithmic distance penalty r1_h ln(1 + r2_h (i - j)) (r1, r2 float32 [n_heads] or nullptr), over a keys-only
// cache entry whose keys are also the values, and an element-wise sigmoid gate (float32 [T, gate_stride] or nullptr).
struct MixedAttention {
    const float *r1 = nullptr, *r2 = nullptr, *mix = nullptr, *gate = nullptr;
    int gate_stride = 0;
};
bool attention_mixed_supported(DType dtype, int nh, int nkv, int d);
Mat attention_mixed(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const MixedAttention& m);
// Differential attention (csrc/attention_diff.cu): every head has two score maps over the same values.  q [T, heads * 2 d]
// (a head's row is [q_1, q_2]), the cache entry's key rows [k_1, k_2] (kv.head_dim == 2 d) and value rows of
// kv.v_head_dim; o = a_1 - lambda a_2, divided by its root mean square over the head's values (eps inside the root), times
// out_scale.  g.head_dim is d, the size of ONE map.  Returns [T, heads * v_head_dim] in q's dtype.
// Kernels: prompts in bfloat16 with d and dv multiples of 16 (d up to 192, dv up to 128) on warp-level MMA; bfloat16
// steps of one token per sequence (d a multiple of 8, dv even) on a kernel that reads every key and value row once for
// the query heads that share it, the keys dealt to attention_diff_splits blocks; everything else (the float32 mode, whose
// sums keep one order) on the plain kernel.
struct DiffAttention {
    float lambda = 0.f, eps = 1e-6f, out_scale = 1.f;
};
// Blocks per (token, group of query heads) of a single-token step: about two per SM in all (a block keeps tens of
// kilobytes of loads in flight), at most one per 256 keys of the longest sequence the cache allows, at most 64.
int attention_diff_splits(long long T, int head_groups, long long max_seq_len, int n_sms);
Mat attention_diff(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const DiffAttention& p);
// Attention of the step's tokens over a cache entry: picks the kernel for the dtype, head size and kind of step.
Mat attention(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale);

// ---- pieces of mixers other than the plain attention

// stream.x <- rmsnorm(alpha * stream.x + delta) * w (w float32, the stream float32); returns the new rows
// in `out_dtype` as well (what the next sublayer reads).
Mat scale_add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& weight_f32, float alpha, float eps, DType out_dtype);

// Between the packed projection x [T, ld] (float32 or the activation dtype) of an attention layer and its attention kernel:
// optional biases, optional RMS norms over a token's whole q and whole k projection, rotation of the
// first `rot_dim` channels of every head (interleaved pairs or rotate-half) from a (cos, sin) table,
// q to a new [T, n_heads * head_dim] matrix of `act_dtype`, k and v into the pages.  k_off < 0: q only.
struct QkPrep {
    int q_off = 0, k_off = -1, v_off = -1;
    const float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr;
    const float *q_norm = nullptr, *k_norm = nullptr;
    float eps = 0.f;
    const float* cos_sin = nullptr;
    int rot_dim = 0;
    bool pairs = false;
    long long n_pos = 0;
    // a temperature on the queries that grows with the position p: q *= 1 + q_temp_coef * ln((p + 1) / q_temp_every + 1)
    // (whole-numbered division), behind the bias; q_temp_every 0: none
    float q_temp_coef = 0.f;
    int q_temp_every = 0;
};
Mat qk_prep(Device& dev, const Mat& x, const QkPrep& p, Geometry g, const StepView& ctx, const KVView& kv, DType act_dtype);

// The decayed linear-attention recurrence over per-sequence state (csrc/decay_state.cu): x_f32 is the
// packed float32 projection (its q, k and v columns are prepared in place), state the cache entry's
// float32 [slots, heads x d x dv] (the kernel's own layout).  Returns float32
// [T, heads * dv].
struct DecayScan {
    int q_off = 0, k_off = 0, v_off = 0;
    int n_heads = 0, head_dim = 0, v_head_dim = 0;
    int qk_act = 0, v_act = 0;          // 0: none, 1: silu
    const float* cos_sin = nullptr;     // rotate-half table or nullptr
    int rot_dim = 0;
    long long n_pos = 0;
    float k_scale = 1.f;
    const float* decay = nullptr;       // float32 [heads] on the device
    // false: a long prompt of few sequences may be cut into segments that run side by side (the order of
    // the sums then differs from token by token); true: always in order, bit for bit
    bool in_order = true;
};
// In how many segments a prompt step's sequences are cut: enough to fill the GPU about twice, at most 8,
// none shorter than 128 tokens; 1 for single tokens.
int decay_scan_segments(int B, int n_heads, int v_head_dim, int max_q, int n_sms);
Mat decay_scan(Device& dev, const Mat& x_f32, const DecayScan& p, const StepView& ctx, const StateView& st);
bool decay_scan_supported(int head_dim, int v_head_dim);
// The same recurrence with a gate pair per token and head in place of the fixed decay: S_t = a_t S_(t-1) + b_t k_t v_t^T,
// o_t = S_t^T q_t; ga, gb float32 [T, n_heads] on the device; n_qk_heads query/key heads shared by n_heads / n_qk_heads
// value heads each; q, k, v are columns of x_f32 and read as they are.  The state block S [n_heads, dv, d] stands at
// the start of the slot's elements (the entry may hold more behind it).  in_order as in DecayScan.
struct GatedScan {
    int q_off = 0, k_off = 0, v_off = 0;
    int n_heads = 0, n_qk_heads = 0, head_dim = 0, v_head_dim = 0;
    const float *ga = nullptr, *gb = nullptr;
    bool in_order = true;
};
Mat gated_scan(Device& dev, const Mat& x_f32, const GatedScan& p, const StepView& ctx, const StateView& st);
// The gates of the matrix memory with exponential gating (csrc/gated_state.cu): from the input and forget logits at
// i_off and f_off of x_f32 (+ biases, soft-capped) and the running maximum and normaliser kept at n_off / m_off of the
// slot's elements, ga, gb and the output factor q_scale / (max(|q_scale n.q|, exp(-m)) + 1e-6), each float32 [T, heads].
struct MlstmGates {
    int q_off = 0, k_off = 0, i_off = 0, f_off = 0;
    const float *i_bias = nullptr, *f_bias = nullptr;
    float cap = 1.f, q_scale = 1.f;
    int n_heads = 0, head_dim = 0;
    long long n_off = 0, m_off = 0;
};
void mlstm_gates(Device& dev, const Mat& x_f32, const MlstmGates& p, const StepView& ctx, const StateView& st, float* ga, float* gb, float* scale);
// dt = softplus(x[dt_off + h] + dt_bias[h]); ga = exp(-exp(a_log[h]) dt); gb = dt
void ssm_gates(Device& dev, const Mat& x_f32, int dt_off, const float* dt_bias, const float* a_log, int n_heads, float* ga, float* gb);
// group_norm_gate with what some recurrences put before the norm: a factor per token and head on o (row_scale
// [T, heads]), a skip term skip_w[head] * skip_x[t, column] (skip_x float32 rows skip_ld apart), and the gate before
// the norm instead of behind it (gate_first)
struct NormGateExtras {
    const float* row_scale = nullptr;
    int head = 0;                 // columns per head
    const float *skip_w = nullptr, *skip_x = nullptr;
    int skip_ld = 0;
    bool gate_first = false;
};
Mat group_norm_gate_ex(Device& dev, const Mat& o_f32, int group, const float* w, int w_len, float eps, const float* gate, int gate_ld, int gate_act,
                       DType out_dtype, const NormGateExtras& ex);
// y = o / sqrt(mean over groups of `group` columns (o^2) + eps) (* w) * act(gate), gate_act 1: silu, 2: sigmoid;
// w has w_len entries (0: the whole row), a shorter one repeats along the row (one group's weight for every group)
Mat group_norm_gate(Device& dev, const Mat& o_f32, int group, const float* w, float eps, const float* gate, int gate_ld, int gate_act,
                    DType out_dtype, int w_len = 0);

// ---- pieces of further mixers, feed-forwards and embeddings

// Activations of the gated feed-forward: act(gate) * up.
// kActSwishClamped (routed experts only): g = min(gate, limit), u = clamp(up, -limit, limit); g sigmoid(1.702 g) (u + 1)
enum GateAct { kActSilu = 1, kActRelu = 2, kActGeluTanh = 3, kActSwishClamped = 4 };
int gate_act_from_name(const std::string& name);        // ConfigError-free: -1 for an unknown name
// resid += d1 (+ d2), all float32 [T, H], and the RMS norm of the new rows times w (float32 [H]) in `out_dtype`: one kernel
Mat add2_rmsnorm(Device& dev, const Mat& resid, const Mat& d1, const Mat* d2, const Mat& weight_f32, float eps, DType out_dtype);
// resid += delta * ls, all float32 (ls float32 [H] on the device), and, with a weight,
// the RMS norm of the new rows times w (float32 [H]) in `out_dtype`: a sublayer's output through a per-channel layer scale,
// folded into the next norm.  Without a weight an empty matrix comes back.
Mat scaled_add_rmsnorm(Device& dev, const Mat& resid, const Mat& delta_f32, const float* ls, const Mat* weight_f32, float eps,
                       DType out_dtype);
// y[t, :] += bias (float32 [cols] on the device), in place
void add_bias(Device& dev, const Mat& y, const float* bias);
// columns [off, off + n) of a float32 matrix as a contiguous matrix of `dtype`
Mat take_columns(Device& dev, const Mat& x_f32, long long off, long long n, DType dtype);
// [a, b] row by row (two float32 matrices of equal shape) as a matrix of `dtype`
Mat join_rows(Device& dev, const Mat& a_f32, const Mat& b_f32, DType dtype);

// Token embedding plus a hashed bigram table (csrc/bigram_embedding.cu); last_token: the int32 per-sequence state.
struct BigramHash { long long buckets = 0, mul_prev = 0, mul_cur = 0; };
Mat bigram_embedding(Device& dev, const StepView& ctx, const Mat& table, const Mat& bigram, const BigramHash& hash, const StateView& last_token);

// The gated delta rule with a decay per head and key channel (csrc/delta_state.cu).  x_f32: the packed float32
// projection with q, k, v and beta's logits at the given columns; a_f32 [T, heads * head_dim]: the decay
// projection.  The state entry holds S and the convolution's rows (delta_rule_state_elements).  Returns float32
// [T, heads * v_head_dim].
struct DeltaRule {
    int q_off = 0, k_off = 0, v_off = 0, b_off = 0;
    int n_heads = 0, n_kv_heads = 0, head_dim = 0, v_head_dim = 0, taps = 1;
    const float *conv_q = nullptr, *conv_k = nullptr, *conv_v = nullptr;     // float32 [channels, taps]
    const float *a_log = nullptr, *dt_bias = nullptr;                        // float32 [heads], [heads * head_dim]
    float q_scale = 1.f;
};
long long delta_rule_state_elements(int n_heads, int n_kv_heads, int head_dim, int v_head_dim, int taps);
bool delta_rule_supported(int head_dim, int v_head_dim, int taps);
Mat delta_rule(Device& dev, const Mat& x_f32, const Mat& a_f32, const DeltaRule& p, const StepView& ctx, const StateView& st);

// Attention through latents (csrc/latent_attention.cu): the two norms and the cache write; returns the normed
// query latent [T, q_rank] in `act_dtype`.  kv: a keys-only entry of one head of kv_rank channels.
Mat latent_prep(Device& dev, const Mat& x_f32, int q_rank, int kv_rank, const float* w_q, const float* w_kv, float eps, const StepView& ctx,
                const KVView& kv, DType act_dtype);
// Attention of `heads` query heads over one shared key/value head of ANY width (a keys-only cache entry), float32 math:
// for widths the framework's attention kernels do not take.  q [T, heads * width] in the cache's dtype.
// gate (float32 [T, gate_stride] or nullptr): head h of token t is multiplied by sigmoid(gate[t * gate_stride + h])
Mat latent_attention_any(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, int heads, float scale, const float* gate = nullptr,
                         int gate_stride = 0);
// y[t, h, :] = W_h x[t, h, :] (transposed = false, w [heads * n_out, n_in]) or W_h^T x[t, h, :] (w [heads * n_in, n_out])
Mat head_linear(Device& dev, const Mat& x, const Mat& w, int heads, bool transposed, DType out_dtype);
// The same where a head's input is the first n_in channels of a wider piece of x (x [T, heads * x_head_stride]) and/or its
// output goes to the first n_out channels of a wider piece of an existing matrix `into` ([T, heads * y_head_stride]).
struct HeadPieces {
    long long x_head_stride = 0;      // 0: n_in
    Mat* into = nullptr;              // nullptr: a new [T, heads * n_out] matrix
    long long y_head_stride = 0;      // with `into`
};
Mat head_linear_pieces(Device& dev, const Mat& x, const Mat& w, int heads, bool transposed, DType out_dtype, const HeadPieces& pc);
// The step between the packed projection and attention of a latent-attention layer with rotated channels
// (latent_rope_prep_kernel, csrc/latent_attention.cu).  x_f32: the packed projection with the queries (heads x (d + dr)) at
// q_off and [latent (kv_rank), raw shared key part (dr)] at c_off.  Writes the cache row [normed latent, rotated key part],
// returns q_nope [T, heads * d] (float32 for single tokens, else the activation dtype) and fills the last dr channels per
// head of qa [T, heads * (kv_rank + dr)] (activation dtype) with the rotated query parts.
struct LatentRope {
    int q_off = 0, c_off = 0, n_heads = 0, head_dim = 0, rot_head_dim = 0, kv_rank = 0;
    const float* w_kv = nullptr;
    float eps = 1e-6f;
    const float* cos_sin = nullptr;
    int rot_dim = 0;
    bool pairs = true;
    long long n_pos = 0;
};
Mat latent_rope_prep(Device& dev, const Mat& x_f32, const LatentRope& p, const StepView& ctx, const KVView& kv, DType act_dtype, Mat* qa);

// Routed feed-forward (csrc/moe.cu).  logits float32 [T, experts] without the bias.  w_gate_up [experts * 2 ff, hidden]
// (per expert, rows 2i and 2i + 1 are gate and up of output i), w_down [experts * hidden, ff].  Returns float32 [T, hidden].
Mat moe_forward(Device& dev, const Mat& h, const Mat& logits_f32, const float* router_bias, int experts, int top, const Mat& w_gate_up,
                const Mat& w_down, int act);
// How the experts are chosen and weighted.  scoring 0: the largest logits (+ bias), weights the softmax over the chosen;
// scoring 1: scores are the softmax over all experts (2: the sigmoid of every logit), `bias` enters the choice only, the
// experts form `groups` equal groups of neighbours of which the `keep` best (by the sum of their `group_top` largest choice
// scores) may be chosen from, and the weights are the chosen scores, divided by their sum (+ sum_eps) only if `renorm`,
// then times weight_scale.  plus: float32 [T, hidden] added to the result.  act_limit: the limit of kActSwishClamped.
struct MoeRouting {
    int scoring = 0, groups = 1, keep = 1, group_top = 1;
    float sum_eps = 0.f, weight_scale = 1.f, act_limit = 0.f;
    bool renorm = true;
    const float* bias = nullptr;
    const Mat* plus = nullptr;
};
Mat moe_forward_ex(Device& dev, const Mat& h, const Mat& logits_f32, const MoeRouting& r, int experts, int top, const Mat& w_gate_up,
                   const Mat& w_down, int act);

// float32 [B, V] -> int32 [B], the lowest id among equal maxima.
int* argmax(Device& dev, const float* logits, long long B, long long V, int* out /* nullptr: from the arena */);
// Temperature / repetition penalty / top-k / top-p sampling, one draw per row (the reference's chain,
// src/utils.cpp:31-115).  uniforms float32 [B] in [0, 1); last_tokens int32 [B, n_last] (-1 pads) or nullptr.
int* sample(Device& dev, const float* logits, long long B, long long V, const float* uniforms, float temp, int top_k, float top_p,
            float repeat_penalty, const int* last_tokens, int n_last, int* out /* nullptr: from the arena */);
void fill_random(Device& dev, void* out, DType dtype, long long n, unsigned long long key, float std, float mean);
void convert(Device& dev, const void* src, DType src_dtype, void* dst, DType dst_dtype, long long n);
// x in another dtype, as a new activation (x itself if it has that dtype already)
Mat cast(Device& dev, const Mat& x, DType dtype);

long long launch_count();               // kernels of this package launched so far (graph replays counted by the engine)
void count_replayed_launches(long long n);
void set_pdl(bool on);

}  // namespace ops
}  // namespace illm
