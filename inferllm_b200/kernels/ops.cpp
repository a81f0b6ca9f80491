#include "kernels/ops.h"

#include <algorithm>
#include <cmath>

#include "csrc/kernels.h"

namespace illm {
namespace ops {

static long long g_replayed = 0;
long long launch_count() { return illm_launch_count() + g_replayed; }
void count_replayed_launches(long long n) { g_replayed += n; }
void set_pdl(bool on) { illm_set_pdl(on ? 1 : 0); }

GemmBackend gemm_backend_from_name(const std::string& name) {
    if (name == "auto") return GemmBackend::Auto;
    if (name == "tc") return GemmBackend::TC;
    if (name == "library") return GemmBackend::Library;
    throw EngineError("gemm backend must be 'tc', 'library' or 'auto', found '" + name + "'");
}
const char* gemm_backend_name(GemmBackend b) { return b == GemmBackend::Auto ? "auto" : b == GemmBackend::TC ? "tc" : "library"; }

static int code_of(DType t, const char* what) {
    if (t == DType::F32) return 0;
    if (t == DType::BF16) return 1;
    throw KernelError(std::string(what) + ": unsupported dtype " + dtype_word(t) + ": the kernels take float32 and bfloat16");
}
static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
static void need(const Mat& m, const char* name, bool want_dtype = false, DType dtype = DType::BF16) {
    if (m.p == nullptr && m.rows * m.cols > 0) throw KernelError(std::string(name) + " has no storage");
    if (want_dtype && m.dtype != dtype)
        throw KernelError(std::string(name) + " must be " + dtype_word(dtype) + ", found " + dtype_word(m.dtype));
    // rows of a multiple of 16 bytes are read 16 bytes at a time
    if (((uintptr_t)m.p & 15) && (m.cols * (long long)dtype_size(m.dtype)) % 16 == 0 && m.rows * m.cols > 0)
        throw KernelError(std::string(name) + " must start on a 16-byte boundary");
}
static void* row_ptr(const Mat& m, long long row) { return (char*)m.p + (size_t)row * m.cols * dtype_size(m.dtype); }

Mat new_mat(Device& dev, long long rows, long long cols, DType dtype) {
    Mat m;
    m.rows = rows;
    m.cols = cols;
    m.dtype = dtype;
    m.rows_held = rows;
    if (dtype == DType::BF16 && rows > kLibraryRowBucket && rows % kLibraryRowBucket)
        m.rows_held = ceil_div(rows, kLibraryRowBucket) * kLibraryRowBucket;
    m.p = dev.alloc((size_t)m.rows_held * cols * dtype_size(dtype));
    return m;
}
static Mat new_mat_exact(Device& dev, long long rows, long long cols, DType dtype) {
    Mat m;
    m.rows = m.rows_held = rows;
    m.cols = cols;
    m.dtype = dtype;
    m.p = dev.alloc((size_t)rows * cols * dtype_size(dtype));
    return m;
}

// ---- policies

int gemm_tc_splits(long long M, long long N, long long K, int n_sms) {
    if (M > 64) return 1;
    const long long tiles = ceil_div(N, 128), k_iters = ceil_div(K, 64);
    long long splits = std::max<long long>(1, std::min<long long>({2LL * n_sms / tiles, k_iters / 8, 8}));   // (more than 8 slices cost their readers more than they win)
    const long long per = ceil_div(k_iters, splits);
    return (int)ceil_div(k_iters, per);          // every slice owns at least one 64-wide piece of K
}

int attention_decode_ring_splits(long long T, int n_kv_heads, long long max_len, int head_dim, int n_sms, double stream_bytes_per_us) {
    const long long pairs = std::max<long long>(1, T * n_kv_heads), tiles = std::max<long long>(1, ceil_div(max_len, 64));
    const long long slots = 2LL * n_sms;
    const double stream_us = (double)pairs * (double)max_len * head_dim * 4 / stream_bytes_per_us;
    int best = 1;
    double best_us = INFINITY;
    for (long long n = 1; n <= std::min<long long>(tiles, kRingDecodeMaxSplits); n++) {
        const long long blocks = pairs * n;
        const double waves = (double)blocks / slots;
        double stretch;
        if (blocks <= slots) {
            stretch = 1.0 / std::min(1.0, blocks / 160.0);
        } else {
            const long long full = blocks / slots, rest = blocks % slots;
            stretch = (full + (rest ? std::max((double)rest / slots, 0.43) : 0.0)) / waves;
        }
        const double us = stream_us * stretch + (n > 1 ? 2.5 + 0.7 * n : 0.0) + 1.0 * ceil_div(blocks, slots);
        if (us < best_us - 1e-9) {
            best = (int)n;
            best_us = us;
        }
    }
    return best;
}

bool attention_decode_ring_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16 && page_size % 64 == 0;
}
bool attention_decode_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && nkv > 0 && nh % nkv == 0 && illm_attention_decode_supported(d, nh / nkv, page_size) != 0;
}
bool attention_decode_gqa_supported(DType dtype, int nh, int nkv, int d) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv >= 2 && nh / nkv <= 16;
}
bool attention_prefill_supported(DType dtype, int nh, int nkv, int d) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0;
}
bool attention_prefill_tc_supported(DType dtype, int nh, int nkv, int d, int page_size) {
    return dtype == DType::BF16 && (d == 64 || d == 128) && nkv > 0 && nh % nkv == 0 && page_size % 64 == 0;
}
std::string attention_kernels_for(DType dtype, int nh, int nkv, int d, int page_size) {
    const int group = nkv ? nh / nkv : 0;
    std::string prompt = attention_prefill_tc_supported(dtype, nh, nkv, d, page_size) ? "prefill_tc (tcgen05)"
                         : attention_prefill_supported(dtype, nh, nkv, d)             ? "prefill (mma.sync)"
                                                                                      : "generic (float32 SIMT, O(T^2) global reads)";
    std::string decode;
    if (attention_decode_ring_supported(dtype, nh, nkv, d, page_size)) decode = "decode_ring (TMA ring)";
    else if ((group >= kGqaDecodeMinGroup || !attention_decode_supported(dtype, nh, nkv, d, page_size)) &&
             attention_decode_gqa_supported(dtype, nh, nkv, d)) decode = "decode_gqa (mma.sync)";
    else if (attention_decode_supported(dtype, nh, nkv, d, page_size)) decode = "decode (split keys)";
    else decode = "generic (float32 SIMT)";
    return "prompts: " + prompt + "; single tokens: " + decode;
}

// ---- element-wise kernels

Mat embedding(Device& dev, const int* ids, long long T, const Mat& table, int* err) {
    need(table, "table");
    Mat out = new_mat_exact(dev, T, table.cols, DType::F32);
    check_kernel(illm_embedding(ids, table.p, code_of(table.dtype, "embedding"), (float*)out.p, (int)T, (int)table.cols, (int)table.rows,
                                err, dev.stream()),
                 "embedding");
    return out;
}

Mat embedding_scaled(Device& dev, const StepView& ctx, const Mat& table, float scale, const float* inv_freq) {
    need(table, "table");
    Mat out = new_mat_exact(dev, ctx.T, table.cols, DType::F32);
    check_kernel(illm_embedding_scaled(ctx.ids, ctx.token_pos, table.p, code_of(table.dtype, "embedding"), (float*)out.p, ctx.T, (int)table.cols,
                                       (int)table.rows, scale, inv_freq, ctx.err, dev.stream()),
                 "embedding_scaled");
    return out;
}

Mat layernorm_sandwich(Device& dev, const Mat& resid, const Mat* delta, const Mat* post_w, const Mat* w, float eps, DType out_dtype, const int* rows,
                       long long n_rows) {
    need(resid, "the residual stream", true, DType::F32);
    const long long H = resid.cols, n = rows ? n_rows : resid.rows;
    if (delta) {
        need(*delta, "the sublayer's output", true, DType::F32);
        if (!post_w || post_w->dtype != DType::F32 || post_w->rows * post_w->cols != H || delta->rows != resid.rows || delta->cols != H)
            throw KernelError("layernorm: the sublayer's output and its norm weight must be float32 of the stream's shape and width");
    }
    if (w && (w->dtype != DType::F32 || w->rows * w->cols != H)) throw KernelError("layernorm: the weight must be float32 of the stream's width");
    if (H > kMaxNormWidth) throw KernelError("layernorm: rows of " + std::to_string(H) + " elements are beyond the kernel");
    Mat y;
    if (w) y = new_mat(dev, n, H, out_dtype);
    check_kernel(illm_layernorm_sandwich((float*)resid.p, delta ? (const float*)delta->p : nullptr, delta ? (const float*)post_w->p : nullptr,
                                         w ? (const float*)w->p : nullptr, w ? y.p : nullptr, w ? code_of(out_dtype, "layernorm") : 0, rows, (int)n,
                                         (int)H, eps, rows == nullptr ? 1 : 0, dev.stream()),
                 "layernorm_sandwich");
    return y;
}

void short_conv(Device& dev, const Mat& x, const ShortConv& p, const StepView& ctx, const StateView& st, const Mat& out, int o_off) {
    need(x, "the convolution's input", true, DType::F32);
    if (p.C <= 0 || p.taps < 1 || p.x_off < 0 || p.x_off + p.C > x.cols || o_off < 0 || o_off + p.C > out.cols || out.rows != x.rows)
        throw KernelError("short_conv: the channels do not lie inside the rows");
    if (p.taps > 1 && (!st.state || st.dtype != DType::F32 || p.state_off < 0 || p.state_off + (long long)(p.taps - 1) * p.C > st.elements))
        throw KernelError("short_conv: the cache entry does not hold the convolution's float32 rows");
    check_kernel(illm_short_conv((const float*)x.p, (int)x.rows, (int)x.cols, p.x_off, p.C, p.taps, p.w, p.bias, p.act, p.residual ? 1 : 0,
                                 (float*)st.state, st.elements, p.state_off, st.slots, ctx.cu_q, ctx.token_seq, ctx.B, out.p,
                                 code_of(out.dtype, "short_conv"), (int)out.cols, o_off, p.update ? 1 : 0, dev.stream()),
                 "short_conv");
}

Mat materialize(Device& dev, const Partials& p, DType dtype) {
    Mat out = new_mat_exact(dev, p.rows, p.cols, dtype);
    check_kernel(illm_splitk_reduce(p.ws, out.p, code_of(dtype, "splitk_reduce"), p.rows * p.cols, p.splits, dev.stream()), "splitk_reduce");
    return out;
}

Mat add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& weight, float eps, DType out_dtype,
                const int* rows, long long n_rows, bool write_resid) {
    need(resid, "resid", true, DType::F32);
    const long long H = resid.cols;
    if (H > kMaxNormWidth)
        throw KernelError("rmsnorm: width " + std::to_string(H) + " exceeds the " + std::to_string(kMaxNormWidth) +
                          " that one block's shared memory holds");
    const Partials* partials = nullptr;
    Mat d;
    bool has_delta = false;
    if (delta && delta->is_partials()) {
        if (out_dtype == DType::BF16 && H % 8 == 0 && H <= 16384 && delta->part.rows == resid.rows && delta->part.cols == resid.cols) {
            partials = &delta->part;
        } else {
            d = materialize(dev, delta->part, out_dtype);
            has_delta = true;
        }
    } else if (delta) {
        d = delta->m;
        has_delta = true;
    }
    if (has_delta) {
        need(d, "delta", true, out_dtype);
        if (d.rows != resid.rows || d.cols != resid.cols)
            throw KernelError("delta [" + std::to_string(d.rows) + ", " + std::to_string(d.cols) + "] does not match resid [" +
                              std::to_string(resid.rows) + ", " + std::to_string(resid.cols) + "]");
    }
    need(weight, "norm weight");
    if (weight.rows * weight.cols != H)
        throw KernelError("norm weight has " + std::to_string(weight.rows * weight.cols) + " elements, the rows have " + std::to_string(H));
    const long long n = rows ? n_rows : resid.rows;
    Mat y = new_mat(dev, n, H, out_dtype);
    if (partials)
        check_kernel(illm_add_rmsnorm_partials((float*)resid.p, partials->ws, partials->splits, partials->rows * partials->cols, weight.p,
                                               code_of(weight.dtype, "rmsnorm"), y.p, code_of(out_dtype, "rmsnorm"), rows, (int)n, (int)H, eps,
                                               write_resid ? 1 : 0, dev.stream()),
                     "add_rmsnorm_partials");
    else
        check_kernel(illm_add_rmsnorm((float*)resid.p, has_delta ? d.p : nullptr, weight.p, code_of(weight.dtype, "rmsnorm"), y.p,
                                      code_of(out_dtype, "rmsnorm"), rows, (int)n, (int)H, eps, write_resid ? 1 : 0, dev.stream()),
                     "add_rmsnorm");
    return y;
}

void residual_add(Device& dev, const Mat& resid, const MatOrPartials& delta) {
    Mat d = delta.is_partials() ? materialize(dev, delta.part, DType::BF16) : delta.m;
    need(resid, "resid", true, DType::F32);
    need(d, "delta");
    if (d.rows != resid.rows || d.cols != resid.cols) throw KernelError("residual_add: shapes differ");
    check_kernel(illm_residual_add((float*)resid.p, d.p, code_of(d.dtype, "residual_add"), resid.rows * resid.cols, dev.stream()),
                 "residual_add");
}

Mat swiglu(Device& dev, const MatOrPartials& gu_in) {
    Mat gu;
    if (gu_in.is_partials()) {
        const Partials& p = gu_in.part;
        if (p.cols % 16 == 0) {
            Mat out = new_mat(dev, p.rows, p.cols / 2, DType::BF16);
            check_kernel(illm_swiglu_partials(p.ws, p.splits, p.rows * p.cols, out.p, (int)p.rows, (int)(p.cols / 2), dev.stream()),
                         "swiglu_partials");
            return out;
        }
        gu = materialize(dev, p, DType::BF16);
    } else {
        gu = gu_in.m;
    }
    need(gu, "gu");
    if (gu.cols % 2) throw KernelError("swiglu: the packed projection must have an even number of columns");
    Mat out = new_mat(dev, gu.rows, gu.cols / 2, gu.dtype);
    check_kernel(illm_swiglu(gu.p, out.p, code_of(gu.dtype, "swiglu"), (int)gu.rows, (int)(gu.cols / 2), dev.stream()), "swiglu");
    return out;
}

// ---- matrix products

Mat gemm_f32(Device& dev, const Mat& x, const Mat& w) {
    need(x, "x", true, DType::F32);
    need(w, "w", true, DType::F32);
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (w.cols != K)
        throw KernelError("gemm: x is [" + std::to_string(M) + ", " + std::to_string(K) + "] but w is [" + std::to_string(w.rows) + ", " +
                          std::to_string(w.cols) + "]");
    Mat out = new_mat_exact(dev, M, N, DType::F32);
    for (long long m0 = 0; m0 < M; m0 += 65535LL * 64) {
        const long long m1 = std::min(M, m0 + 65535LL * 64);
        check_kernel(illm_gemm_f32_nt((const float*)row_ptr(x, m0), (const float*)w.p, (float*)row_ptr(out, m0), (int)(m1 - m0), (int)N, (int)K,
                                      (int)K, (int)K, (int)N, dev.tc_error_word(), dev.stream()),
                     "gemm_f32");
    }
    return out;
}

static void check_product(const Mat& x, const Mat& w, const char* what, bool gated = false) {
    need(x, "x", true, DType::BF16);
    need(w, "w", true, DType::BF16);
    if (w.cols != x.cols)
        throw KernelError("gemm: x is [" + std::to_string(x.rows) + ", " + std::to_string(x.cols) + "] but w is [" + std::to_string(w.rows) +
                          ", " + std::to_string(w.cols) + "]");
    if (x.cols % 8 || ((uintptr_t)x.p & 15) || ((uintptr_t)w.p & 15) || (gated && w.rows % 2))
        throw KernelError(std::string(what) + ": K = " + std::to_string(x.cols) +
                          " must be a multiple of 8, the operands 16-byte aligned and a gated weight an even number of rows");
}

MatOrPartials gemm_bf16_tc(Device& dev, const Mat& x, const Mat& w, DType out_dtype, int splits, bool defer_reduce) {
    check_product(x, w, "gemm_bf16_tc");
    const long long M = x.rows, K = x.cols, N = w.rows;
    MatOrPartials r;
    r.m = new_mat_exact(dev, M, N, out_dtype);
    if (splits <= 0) {
        splits = gemm_tc_splits(M, N, K, dev.n_sms());
    } else {
        const long long k_iters = ceil_div(K, 64);
        long long s = std::max<long long>(1, std::min<long long>(splits, k_iters));
        splits = (int)ceil_div(k_iters, ceil_div(k_iters, s));
    }
    if (M > 64) splits = 1;
    float* ws = splits > 1 ? dev.alloc_n<float>((size_t)splits * M * N) : nullptr;
    const bool defer = defer_reduce && splits > 1;
    check_kernel(illm_gemm_bf16_tc(x.p, w.p, r.m.p, code_of(out_dtype, "gemm_bf16_tc"), (int)M, (int)N, (int)K, ws, splits, dev.tc_error_word(),
                                   dev.stream(), defer ? 1 : 0),
                 "gemm_bf16_tc");
    if (defer) {
        r.part.ws = ws;
        r.part.splits = splits;
        r.part.rows = M;
        r.part.cols = N;
    }
    return r;
}

Mat gemm_bf16_tc2(Device& dev, const Mat& x, const Mat& w, DType out_dtype, bool gated, int act) {
    check_product(x, w, "gemm_bf16_tc2", gated);
    const long long M = x.rows, K = x.cols, N = w.rows;
    Mat out = new_mat(dev, M, gated ? N / 2 : N, out_dtype);
    check_kernel(illm_gemm_bf16_tc2(x.p, w.p, out.p, code_of(out_dtype, "gemm_bf16_tc2"), gated ? act : 0, (int)M, (int)N, (int)K,
                                    dev.tc_error_word(), dev.stream()),
                 "gemm_bf16_tc2");
    return out;
}

MatOrPartials linear(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, DType out_dtype, bool defer_reduce) {
    MatOrPartials r;
    if (x.dtype == DType::F32) {
        r.m = gemm_f32(dev, x, w);
        return r;
    }
    need(x, "x", true, DType::BF16);
    need(w, "w", true, DType::BF16);
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (M > 0 && K % 8 == 0 && (backend == GemmBackend::TC || (backend == GemmBackend::Auto && M <= kGemmTcMaxTokensAuto))) {
        if (M > 128 && N >= 256) {
            r.m = gemm_bf16_tc2(dev, x, w, out_dtype, false);     // prompts: pairs of SMs
            return r;
        }
        return gemm_bf16_tc(dev, x, w, out_dtype, 0, defer_reduce);
    }
    if (w.cols != K) throw KernelError("gemm: the operands' inner sizes differ");
    // the library sees whole buckets of rows where the activation was allocated so (see Mat::rows_held);
    // the rows beyond M are never initialised and never read back: a row of a product depends on its
    // own row of the input only
    long long Mlib = M;
    if (M > kLibraryRowBucket && M % kLibraryRowBucket && x.rows_held >= ceil_div(M, kLibraryRowBucket) * kLibraryRowBucket)
        Mlib = ceil_div(M, kLibraryRowBucket) * kLibraryRowBucket;
    r.m = new_mat_exact(dev, Mlib, N, out_dtype);
    r.m.rows = M;
    if (M > 0) dev.library_gemm_bf16(x.p, w.p, r.m.p, out_dtype, (int)Mlib, (int)N, (int)K);
    return r;
}

Mat linear_gated(Device& dev, GemmBackend backend, const Mat& x, const Mat& w, int act) {
    if (act < kActSilu || act > kActGeluTanh) throw KernelError("linear_gated: unknown activation");
    const long long M = x.rows, K = x.cols, N = w.rows;
    if (x.dtype == DType::BF16 && w.dtype == DType::BF16 && M > 0 && K % 8 == 0 && N % 2 == 0 && !((uintptr_t)x.p & 15) &&
        !((uintptr_t)w.p & 15)) {
        const bool tc = backend == GemmBackend::TC || (backend == GemmBackend::Auto && M <= kGemmTcMaxTokensAuto);
        if (tc && M <= 64 && gemm_tc_splits(M, N, K, dev.n_sms()) == 1) {
            check_product(x, w, "gemm_bf16_tc_gated", true);
            Mat out = new_mat_exact(dev, M, N / 2, DType::BF16);
            check_kernel(illm_gemm_bf16_tc_gated(x.p, w.p, out.p, (int)M, (int)N, (int)K, act, dev.tc_error_word(), dev.stream()),
                         "gemm_bf16_tc_gated");
            return out;
        }
        if (N >= 256 && ((backend == GemmBackend::TC && M > 128) || (backend == GemmBackend::Auto && M >= kGatedPromptsOnTcMinTokens)))
            return gemm_bf16_tc2(dev, x, w, DType::BF16, true, act);
    }
    if (act == kActSilu) return swiglu(dev, linear(dev, backend, x, w, x.dtype, true));
    Mat gu = linear(dev, backend, x, w, x.dtype, false).m;
    if (gu.cols % 2) throw KernelError("gated activation: the packed projection must have an even number of columns");
    Mat out = new_mat(dev, gu.rows, gu.cols / 2, gu.dtype);
    check_kernel(illm_gated_act(gu.p, out.p, code_of(gu.dtype, "gated_act"), (int)gu.rows, (int)(gu.cols / 2), act, dev.stream()), "gated_act");
    return out;
}

// ---- rotation and attention

static void check_cache(const KVView& kv, DType want, Geometry g, const char* what) {
    if (kv.k == nullptr || kv.v == nullptr) throw KernelError(std::string(what) + ": the cache entry has no storage");
    if (kv.dtype != want)
        throw KernelError(std::string(what) + ": the cache pages must be " + dtype_word(want) + ", found " + dtype_word(kv.dtype));
    if (kv.n_kv_heads != g.n_kv_heads || kv.head_dim != g.head_dim)
        throw KernelError(std::string(what) + ": cache pages of " + std::to_string(kv.n_kv_heads) + " heads of " + std::to_string(kv.head_dim) +
                          " do not match the layer's " + std::to_string(g.n_kv_heads) + " heads of " + std::to_string(g.head_dim));
    if (((uintptr_t)kv.k & 15) || ((uintptr_t)kv.v & 15)) throw KernelError(std::string(what) + ": the cache pages must be 16-byte aligned");
}

Mat rope_kv_write(Device& dev, const MatOrPartials& in, const float* cos_sin, int rot_dim, long long n_pos, const StepView& ctx,
                  const KVView& kv, Geometry g) {
    const Partials* partials = nullptr;
    Mat qkv;
    if (in.is_partials()) {
        if (g.head_dim % 8 == 0 && rot_dim % 16 == 0 && kv.writes && kv.k && kv.dtype == DType::BF16) {
            partials = &in.part;
            qkv = new_mat_exact(dev, in.part.rows, in.part.cols, DType::BF16);
        } else {
            qkv = materialize(dev, in.part, DType::BF16);
        }
    } else {
        qkv = in.m;
    }
    need(qkv, "qkv");
    const long long T = qkv.rows;
    if (qkv.cols != (long long)(g.n_heads + 2 * g.n_kv_heads) * g.head_dim)
        throw KernelError("qkv width " + std::to_string(qkv.cols) + " is not (heads + 2 kv heads) * head_dim");
    if (kv.writes) check_cache(kv, qkv.dtype, g, "rope_kv_write");
    if (rot_dim && !cos_sin) throw KernelError("rope_kv_write: a rotation needs its cos/sin table");
    void* kc = kv.writes ? kv.k : nullptr;
    void* vc = kv.writes ? kv.v : nullptr;
    const int code = code_of(qkv.dtype, "rope_kv_write");
    if (partials)
        check_kernel(illm_rope_kv_write_partials(qkv.p, partials->ws, partials->splits, partials->rows * partials->cols, rot_dim ? cos_sin : nullptr,
                                                 ctx.token_pos, ctx.token_seq, kv.block_table, kv.width, kc, vc, code, (int)T, g.n_heads,
                                                 g.n_kv_heads, g.head_dim, rot_dim, kv.page_size, kv.writes ? 1 : 0, (int)(rot_dim ? n_pos : 0),
                                                 ctx.err, dev.stream()),
                     "rope_kv_write_partials");
    else
        check_kernel(illm_rope_kv_write(qkv.p, rot_dim ? cos_sin : nullptr, ctx.token_pos, ctx.token_seq, kv.block_table, kv.width, kc, vc, code,
                                        (int)T, g.n_heads, g.n_kv_heads, g.head_dim, rot_dim, kv.page_size, kv.writes ? 1 : 0,
                                        (int)(rot_dim ? n_pos : 0), ctx.err, dev.stream()),
                     "rope_kv_write");
    return qkv;
}

Mat attention_generic(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                      const AttentionExtras* extras) {
    const int dv = kv.v_head_dim > 0 ? kv.v_head_dim : g.head_dim;
    if (g.head_dim <= 0 || g.head_dim > kMaxHeadDimGeneric || dv > kMaxHeadDimGeneric)
        throw KernelError("attention: head size " + std::to_string(g.head_dim) + " (values " + std::to_string(dv) +
                          ") is not supported (up to " + std::to_string(kMaxHeadDimGeneric) + ")");
    if (g.n_kv_heads <= 0 || g.n_heads % g.n_kv_heads) throw KernelError("attention: heads must be a multiple of kv heads");
    need(qkv, "qkv");
    check_cache(kv, qkv.dtype, g, "attention_generic");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * dv, qkv.dtype);
    check_kernel(illm_attention_generic(qkv.p, (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p,
                                        code_of(qkv.dtype, "attention_generic"), (int)qkv.rows, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size,
                                        kv.window, scale, dv, extras ? extras->sinks : nullptr, extras ? extras->gate : nullptr,
                                        extras ? extras->gate_stride : 0, dev.stream()),
                 "attention_generic");
    return out;
}

// ---- pieces of mixers other than the plain attention

Mat scale_add_rmsnorm(Device& dev, const Mat& resid, const MatOrPartials* delta, const Mat& w, float alpha, float eps, DType out_dtype) {
    need(resid, "resid", true, DType::F32);
    need(w, "norm weight", true, DType::F32);
    const long long H = resid.cols;
    if (w.rows * w.cols != H)
        throw KernelError("norm weight has " + std::to_string(w.rows * w.cols) + " elements, the rows have " + std::to_string(H));
    const Partials* part = delta && delta->is_partials() ? &delta->part : nullptr;
    const Mat* d = delta && !delta->is_partials() ? &delta->m : nullptr;
    if (d) need(*d, "delta");
    if ((d && (d->rows != resid.rows || d->cols != H)) || (part && (part->rows != resid.rows || part->cols != H)))
        throw KernelError("scale_add_rmsnorm: delta does not match the stream");
    Mat y = new_mat(dev, resid.rows, H, out_dtype);
    check_kernel(illm_scale_add_rmsnorm((float*)resid.p, d ? d->p : nullptr, d ? code_of(d->dtype, "scale_add_rmsnorm") : 0, (const float*)w.p, y.p,
                                        code_of(out_dtype, "scale_add_rmsnorm"), (int)resid.rows, (int)H, alpha, eps, part ? part->ws : nullptr,
                                        part ? part->splits : 0, part ? part->rows * part->cols : 0, dev.stream()),
                 "scale_add_rmsnorm");
    return y;
}

Mat qk_prep(Device& dev, const Mat& x, const QkPrep& p, Geometry g, const StepView& ctx, const KVView& kv, DType act_dtype) {
    need(x, "the packed projection");
    if (x.dtype != DType::F32 && x.dtype != act_dtype) throw KernelError("qk_prep: the projection must be float32 or the activation dtype");
    const bool has_kv = p.k_off >= 0;
    const int dv = kv.v_head_dim > 0 ? kv.v_head_dim : g.head_dim;
    const bool store = has_kv && kv.writes;
    if (store) check_cache(kv, act_dtype, g, "qk_prep");
    if (p.rot_dim && !p.cos_sin) throw KernelError("qk_prep: a rotation needs its cos/sin table");
    Mat q = new_mat(dev, x.rows, (long long)g.n_heads * g.head_dim, act_dtype);
    if (p.q_temp_every < 0) throw KernelError("qk_prep: the query temperature's period must not be negative");
    check_kernel(illm_qk_prep_ex(x.p, code_of(x.dtype, "qk_prep"), (int)x.cols, p.q_off, has_kv ? p.k_off : -1, p.v_off, g.n_heads, g.n_kv_heads, g.head_dim, dv,
                                 p.q_bias, p.k_bias, p.v_bias, p.q_norm, p.k_norm, p.eps, p.cos_sin, p.rot_dim, p.pairs ? 1 : 0, (int)p.n_pos,
                                 ctx.token_pos, ctx.token_seq, kv.block_table, kv.width, kv.page_size, q.p, store ? kv.k : nullptr,
                                 store ? kv.v : nullptr, code_of(act_dtype, "qk_prep"), (int)x.rows, ctx.err, p.q_temp_coef, p.q_temp_every, dev.stream()),
                 "qk_prep");
    return q;
}

bool decay_scan_supported(int d, int dv) { return illm_decay_scan_supported(d, dv) != 0; }      // head sizes up to 1024

int decay_scan_segments(int B, int n_heads, int v_head_dim, int max_q, int n_sms) {
    const long long blocks = (long long)B * n_heads * ceil_div(v_head_dim, 64);      // a block covers 64 columns of a head
    long long P = std::min<long long>(8, (4LL * n_sms) / std::max<long long>(blocks, 1));
    P = std::min<long long>(P, max_q / 128);
    return P < 2 ? 1 : (int)P;
}

Mat decay_scan(Device& dev, const Mat& x, const DecayScan& p, const StepView& ctx, const StateView& st) {
    need(x, "the packed projection", true, DType::F32);
    if (!st.state || st.dtype != DType::F32 || st.elements != (long long)p.n_heads * p.head_dim * p.v_head_dim)
        throw KernelError("decay_scan: the cache entry does not hold float32 state of heads x head size x value size");
    if (!decay_scan_supported(p.head_dim, p.v_head_dim))
        throw KernelError("decay_scan: a state of " + std::to_string(p.head_dim) + " x " + std::to_string(p.v_head_dim) +
                          " per head is beyond the kernel (head sizes up to 1024)");
    Mat out = new_mat_exact(dev, x.rows, (long long)p.n_heads * p.v_head_dim, DType::F32);
    const int segments = (p.in_order || ctx.is_decode) ? 1 : decay_scan_segments(ctx.B, p.n_heads, p.v_head_dim, ctx.max_q, dev.n_sms());
    float* seg_state = segments > 1 ? dev.alloc_n<float>((size_t)ctx.B * segments * p.n_heads * p.head_dim * p.v_head_dim) : nullptr;
    check_kernel(illm_decay_scan((float*)x.p, (int)x.rows, (int)x.cols, p.q_off, p.k_off, p.v_off, p.n_heads, p.head_dim, p.v_head_dim, p.qk_act, p.v_act,
                                 p.rot_dim ? p.cos_sin : nullptr, p.rot_dim, (int)p.n_pos, p.k_scale, p.decay, (float*)st.state, st.slots, ctx.cu_q,
                                 ctx.token_pos, (float*)out.p, ctx.B, ctx.err, segments, seg_state, dev.stream()),
                 "decay_scan");
    return out;
}

Mat gated_scan(Device& dev, const Mat& x, const GatedScan& p, const StepView& ctx, const StateView& st) {
    need(x, "the packed projection", true, DType::F32);
    if (p.n_heads <= 0 || p.n_qk_heads <= 0 || p.n_heads % p.n_qk_heads) throw KernelError("gated_scan: the heads must be a multiple of the query/key heads");
    if (!st.state || st.dtype != DType::F32 || st.elements < (long long)p.n_heads * p.head_dim * p.v_head_dim)
        throw KernelError("gated_scan: the cache entry does not hold float32 state of heads x head size x value size");
    if (!decay_scan_supported(p.head_dim, p.v_head_dim)) throw KernelError("gated_scan: the head size is beyond the kernel (up to 1024)");
    Mat out = new_mat_exact(dev, x.rows, (long long)p.n_heads * p.v_head_dim, DType::F32);
    const int segments = (p.in_order || ctx.is_decode) ? 1 : decay_scan_segments(ctx.B, p.n_heads, p.v_head_dim, ctx.max_q, dev.n_sms());
    float* seg_state = segments > 1 ? dev.alloc_n<float>((size_t)ctx.B * segments * p.n_heads * p.head_dim * p.v_head_dim) : nullptr;
    float* seg_gate = segments > 1 ? dev.alloc_n<float>((size_t)ctx.B * segments * p.n_heads) : nullptr;
    check_kernel(illm_gated_scan((const float*)x.p, (int)x.rows, (int)x.cols, p.q_off, p.k_off, p.v_off, p.n_heads, p.n_heads / p.n_qk_heads, p.head_dim,
                                 p.v_head_dim, p.ga, p.gb, (float*)st.state, st.elements, st.slots, ctx.cu_q, (float*)out.p, ctx.B, segments, seg_state, seg_gate,
                                 dev.stream()),
                 "gated_scan");
    return out;
}

void mlstm_gates(Device& dev, const Mat& x, const MlstmGates& p, const StepView& ctx, const StateView& st, float* ga, float* gb, float* scale) {
    need(x, "the packed projection", true, DType::F32);
    if (!st.state || st.dtype != DType::F32 || p.n_off < 0 || p.m_off < 0 || p.n_off + (long long)p.n_heads * p.head_dim > st.elements ||
        p.m_off + p.n_heads > st.elements)
        throw KernelError("mlstm_gates: the cache entry does not hold the normaliser and the running maximum");
    check_kernel(illm_mlstm_gates((const float*)x.p, (int)x.rows, (int)x.cols, p.q_off, p.k_off, p.i_off, p.f_off, p.i_bias, p.f_bias, p.cap, p.q_scale,
                                  p.n_heads, p.head_dim, (float*)st.state, st.elements, p.n_off, p.m_off, st.slots, ctx.cu_q, ga, gb, scale, ctx.B,
                                  dev.stream()),
                 "mlstm_gates");
}

void ssm_gates(Device& dev, const Mat& x, int dt_off, const float* dt_bias, const float* a_log, int n_heads, float* ga, float* gb) {
    need(x, "the packed projection", true, DType::F32);
    check_kernel(illm_ssm_gates((const float*)x.p, (int)x.rows, (int)x.cols, dt_off, dt_bias, a_log, n_heads, ga, gb, dev.stream()), "ssm_gates");
}

Mat group_norm_gate_ex(Device& dev, const Mat& o, int group, const float* w, int w_len, float eps, const float* gate, int gate_ld, int gate_act,
                       DType out_dtype, const NormGateExtras& ex) {
    need(o, "the recurrence's output", true, DType::F32);
    Mat y = new_mat(dev, o.rows, o.cols, out_dtype);
    check_kernel(illm_group_norm_gate_ex((const float*)o.p, (int)o.rows, (int)o.cols, group, w, w_len > 0 ? w_len : (int)o.cols, eps, gate, gate_ld, gate_act,
                                         ex.gate_first ? 1 : 0, ex.row_scale, ex.head, ex.skip_w, ex.skip_x, ex.skip_ld, y.p,
                                         code_of(out_dtype, "group_norm_gate"), dev.stream()),
                 "group_norm_gate");
    return y;
}

bool attention_mixed_supported(DType dtype, int nh, int nkv, int d) {
    return (dtype == DType::F32 || dtype == DType::BF16) && illm_attention_mixed_supported(nh, nkv, d, (int)dtype_size(dtype)) != 0;
}

Mat attention_mixed(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const MixedAttention& m) {
    need(q, "q");
    if (kv.dtype != q.dtype || kv.n_kv_heads != g.n_kv_heads || kv.head_dim != g.head_dim || kv.v != kv.k)
        throw KernelError("attention_mixed: needs a keys-only cache entry of this layer's head count and size, in the activation dtype");
    if (!attention_mixed_supported(q.dtype, g.n_heads, g.n_kv_heads, g.head_dim))
        throw KernelError("attention_mixed: " + std::to_string(g.n_heads) + " heads of " + std::to_string(g.head_dim) + " channels are beyond the kernel");
    if (q.cols < (long long)g.n_heads * g.head_dim) throw KernelError("attention_mixed: q is narrower than heads x head size");
    Mat out = new_mat(dev, q.rows, (long long)g.n_heads * g.head_dim, q.dtype);
    // Prompts and their portions in bfloat16: 16 tokens of a sequence per block, the two products on tensor cores.
    if (q.dtype == DType::BF16 && q.rows > 64 && q.cols % 8 == 0 && (!m.gate || m.gate_stride % 2 == 0) &&
        illm_attention_mixed_tc_supported(g.n_heads, g.n_kv_heads, g.head_dim)) {
        check_kernel(illm_attention_mixed_tc(q.p, (int)q.cols, kv.k, kv.block_table, kv.width, ctx.token_pos, ctx.cu_q, ctx.B, out.p, (int)q.rows, g.n_heads,
                                             g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, m.r1, m.r2, m.mix, m.gate, m.gate_stride,
                                             dev.n_sms(), dev.stream()),
                     "attention_mixed_tc");
        return out;
    }
    // Few tokens over many keys (single-token steps): the keys in parts, so that the step fills the GPU.  How many
    // depends on the step's shape and the cache's limits alone, never on a sequence's length, so that a captured
    // step can be replayed.  The float32 mode keeps one part: its sums have one order for every step.
    int splits = 1;
    float* part = nullptr;
    if (q.dtype != DType::F32 && q.rows <= 64) {
        const long long span = kv.window > 0 && kv.window < ctx.max_seq_len ? kv.window : ctx.max_seq_len;
        const int kt = illm_attention_mixed_keys_per_tile(g.n_heads, g.n_kv_heads, g.head_dim, (int)dtype_size(q.dtype), m.mix != nullptr);
        const long long by_keys = (span + 2 * kt - 1) / (2 * kt), by_blocks = std::max<long long>(1, 2LL * dev.n_sms() / q.rows);
        splits = (int)std::max<long long>(1, std::min(by_keys, by_blocks));
        if (splits > 1) part = dev.alloc_n<float>((size_t)q.rows * splits * ((size_t)g.n_heads * g.head_dim + 2 * g.n_heads));
    }
    check_kernel(illm_attention_mixed(q.p, (int)q.cols, kv.k, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p, code_of(q.dtype, "attention_mixed"),
                                      (int)q.rows, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, m.r1, m.r2, m.mix, m.gate,
                                      m.gate_stride, splits, part, dev.stream()),
                 "attention_mixed");
    return out;
}

Mat group_norm_gate(Device& dev, const Mat& o, int group, const float* w, float eps, const float* gate, int gate_ld, int gate_act,
                    DType out_dtype, int w_len) {
    need(o, "the recurrence's output", true, DType::F32);
    Mat y = new_mat(dev, o.rows, o.cols, out_dtype);
    check_kernel(illm_group_norm_gate((const float*)o.p, (int)o.rows, (int)o.cols, group, w, w_len > 0 ? w_len : (int)o.cols, eps, gate, gate_ld, gate_act, y.p,
                                      code_of(out_dtype, "group_norm_gate"), dev.stream()),
                 "group_norm_gate");
    return y;
}

typedef int (*DecodeFn)(const void*, int, const void*, const void*, const int*, int, const int*, const int*, float*, float*, void*, int, int,
                        int, int, int, int, float, int, void*);

static Mat decode_chunked(Device& dev, DecodeFn fn, const char* what, int chunk_keys, const Mat& qkv, const KVView& kv, const StepView& ctx,
                          Geometry g, float scale, long long max_len) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, what);
    const long long T = qkv.rows;
    const int n_chunks = (int)std::max<long long>(1, ceil_div(max_len, chunk_keys));
    float* part_acc = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * g.head_dim);
    float* part_ml = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * 2);
    Mat out = new_mat(dev, T, (long long)g.n_heads * g.head_dim, DType::BF16);
    for (long long t0 = 0; t0 < T; t0 += 65535) {
        const long long t1 = std::min(T, t0 + 65535);
        check_kernel(fn(row_ptr(qkv, t0), (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos + t0, ctx.token_seq + t0,
                        part_acc + (size_t)t0 * g.n_heads * n_chunks * g.head_dim, part_ml + (size_t)t0 * g.n_heads * n_chunks * 2, row_ptr(out, t0),
                        (int)(t1 - t0), g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n_chunks, dev.stream()),
                     what);
    }
    return out;
}

Mat attention_decode(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len) {
    return decode_chunked(dev, illm_attention_decode, "attention_decode", kDecodeChunk, qkv, kv, ctx, g, scale, max_len);
}
Mat attention_decode_gqa(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len) {
    return decode_chunked(dev, illm_attention_decode_gqa, "attention_decode_gqa", kGqaDecodeChunk, qkv, kv, ctx, g, scale, max_len);
}

Mat attention_decode_ring(Device& dev, const MatOrPartials& in, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                          long long max_len, int splits, const FusedRope* rope, const AttentionExtras* extras) {
    if (rope && extras) throw KernelError("attention_decode_ring: sinks and gates do not go with the fused position encoding");
    long long T, width;
    if (in.is_partials()) {
        if (!rope) throw KernelError("attention_decode_ring: unreduced slices need the fused position encoding");
        T = in.part.rows;
        width = in.part.cols;
    } else {
        need(in.m, "qkv", true, DType::BF16);
        T = in.m.rows;
        width = in.m.cols;
    }
    check_cache(kv, DType::BF16, g, "attention_decode_ring");
    if (rope && width != (long long)(g.n_heads + 2 * g.n_kv_heads) * g.head_dim)
        throw KernelError("qkv width " + std::to_string(width) + " is not (heads + 2 kv heads) * head_dim");
    Mat out = new_mat_exact(dev, T, (long long)g.n_heads * g.head_dim, DType::BF16);
    for (long long t0 = 0; t0 < T; t0 += 65535) {
        const long long t1 = std::min(T, t0 + 65535);
        const int n = splits > 0 ? splits : attention_decode_ring_splits(t1 - t0, g.n_kv_heads, max_len, g.head_dim, dev.n_sms(), dev.stream_bytes_per_us());
        float *part_acc = nullptr, *part_ml = nullptr;
        if (n > 1) {
            part_acc = dev.alloc_n<float>((size_t)(t1 - t0) * g.n_heads * n * g.head_dim);
            part_ml = dev.alloc_n<float>((size_t)(t1 - t0) * g.n_heads * n * 2);
        }
        if (extras) {
            check_kernel(illm_attention_decode_ring_ex(row_ptr(in.m, t0), (int)width, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width,
                                                       ctx.token_pos + t0, ctx.token_seq + t0, part_acc, part_ml, row_ptr(out, t0), (int)(t1 - t0),
                                                       g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n, dev.tc_error_word(),
                                                       extras->wide_weights ? 1 : 0, extras->sinks,
                                                       extras->gate ? extras->gate + (size_t)t0 * extras->gate_stride : nullptr, extras->gate_stride,
                                                       dev.stream()),
                         "attention_decode_ring");
            continue;
        }
        if (!rope) {
            check_kernel(illm_attention_decode_ring(row_ptr(in.m, t0), (int)width, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width,
                                                    ctx.token_pos + t0, ctx.token_seq + t0, part_acc, part_ml, row_ptr(out, t0), (int)(t1 - t0),
                                                    g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n, dev.tc_error_word(),
                                                    dev.stream()),
                         "attention_decode_ring");
            continue;
        }
        if (rope->rot_dim && !rope->cos_sin) throw KernelError("attention_decode_ring: a rotation needs its cos/sin table");
        if (T > 65535) throw KernelError("attention_decode_ring with the position encoding inside takes at most 65535 tokens");
        check_kernel(illm_attention_decode_ring_rope(in.is_partials() ? nullptr : in.m.p, in.is_partials() ? in.part.ws : nullptr,
                                                     in.is_partials() ? in.part.splits : 0, in.is_partials() ? T * width : 0,
                                                     rope->rot_dim ? rope->cos_sin : nullptr, rope->rot_dim, (int)(rope->rot_dim ? rope->n_pos : 0),
                                                     rope->write_kv ? 1 : 0, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width, ctx.token_pos,
                                                     ctx.token_seq, part_acc, part_ml, out.p, (int)T, g.n_heads, g.n_kv_heads, g.head_dim,
                                                     kv.page_size, kv.window, scale, n, dev.tc_error_word(), rope->step_err, dev.stream()),
                     "attention_decode_ring_rope");
    }
    return out;
}

Mat attention_prefill(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, "attention_prefill");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * g.head_dim, DType::BF16);
    check_kernel(illm_attention_prefill(qkv.p, (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.cu_q, ctx.seq_lens, out.p, ctx.B, ctx.max_q,
                                        g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, dev.stream()),
                 "attention_prefill");
    return out;
}

Mat attention_prefill_tc(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale,
                         const AttentionExtras* ex) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, "attention_prefill_tc");
    Mat out = new_mat(dev, qkv.rows, (long long)g.n_heads * g.head_dim, DType::BF16);
    check_kernel(illm_attention_prefill_tc_ex(qkv.p, (int)qkv.cols, (int)qkv.rows, kv.k, kv.v, kv.num_pages, kv.block_table, kv.width, ctx.cu_q,
                                              ctx.seq_lens, out.p, ctx.B, ctx.max_q, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window,
                                              scale, dev.tc_error_word(), ex && ex->wide_weights ? 1 : 0, ex ? ex->sinks : nullptr,
                                              ex ? ex->gate : nullptr, ex ? ex->gate_stride : 0, dev.stream()),
                 "attention_prefill_tc");
    return out;
}

Mat attention_decode_ex(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale, long long max_len,
                        const AttentionExtras& ex) {
    need(qkv, "qkv", true, DType::BF16);
    check_cache(kv, DType::BF16, g, "attention_decode");
    const long long T = qkv.rows;
    if (T > 65535) throw KernelError("attention_decode with sinks or gates takes at most 65535 tokens");
    const int n_chunks = (int)std::max<long long>(1, ceil_div(max_len, kDecodeChunk));
    float* part_acc = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * g.head_dim);
    float* part_ml = dev.alloc_n<float>((size_t)T * g.n_heads * n_chunks * 2);
    Mat out = new_mat(dev, T, (long long)g.n_heads * g.head_dim, DType::BF16);
    check_kernel(illm_attention_decode_ex(qkv.p, (int)qkv.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, part_acc, part_ml,
                                          out.p, (int)T, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size, kv.window, scale, n_chunks, ex.sinks,
                                          ex.gate, ex.gate_stride, dev.stream()),
                 "attention_decode");
    return out;
}

Mat attention_ex(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const AttentionExtras& ex) {
    const int dv = kv.v_head_dim > 0 ? kv.v_head_dim : g.head_dim;
    if (q.dtype == DType::BF16 && dv == g.head_dim) {
        if (ctx.is_decode && attention_decode_ring_supported(q.dtype, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size)) {
            MatOrPartials in;
            in.m = q;
            return attention_decode_ring(dev, in, kv, ctx, g, scale, ctx.max_seq_len, 0, nullptr, &ex);
        }
        if (ctx.is_decode && attention_decode_supported(q.dtype, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size))
            return attention_decode_ex(dev, q, kv, ctx, g, scale, ctx.max_seq_len, ex);
        if (!ctx.is_decode && attention_prefill_tc_supported(q.dtype, g.n_heads, g.n_kv_heads, g.head_dim, kv.page_size))
            return attention_prefill_tc(dev, q, kv, ctx, g, scale, &ex);
    }
    return attention_generic(dev, q, kv, ctx, g, scale, &ex);
}

Mat attention_diff(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, Geometry g, float scale, const DiffAttention& p) {
    need(q, "q");
    const int dv = kv.v_head_dim > 0 ? kv.v_head_dim : kv.head_dim;
    if (g.n_kv_heads <= 0 || g.n_heads % g.n_kv_heads) throw KernelError("attention_diff: heads must be a multiple of kv heads");
    if (g.head_dim <= 0 || g.head_dim > kMaxHeadDimGeneric || dv > kMaxHeadDimGeneric)
        throw KernelError("attention_diff: a score map of " + std::to_string(g.head_dim) + " channels (values " + std::to_string(dv) +
                          ") is not supported (up to " + std::to_string(kMaxHeadDimGeneric) + ")");
    if (!kv.k || !kv.v || kv.dtype != q.dtype || kv.n_kv_heads != g.n_kv_heads || kv.head_dim != 2 * g.head_dim || q.cols < (long long)g.n_heads * 2 * g.head_dim)
        throw KernelError("attention_diff: the cache entry must hold key rows of two maps (2 x " + std::to_string(g.head_dim) + " channels) in the queries' dtype");
    Mat out = new_mat(dev, q.rows, (long long)g.n_heads * dv, q.dtype);
    if (q.dtype == DType::BF16 && !ctx.is_decode && illm_attention_diff_mma_supported(g.head_dim, dv) && q.cols % 8 == 0) {
        check_kernel(illm_attention_diff_mma(q.p, (int)q.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.cu_q, ctx.seq_lens, out.p, ctx.B, ctx.max_q, g.n_heads,
                                             g.n_kv_heads, g.head_dim, dv, kv.page_size, kv.window, scale, p.lambda, p.eps, p.out_scale, dev.stream()),
                     "attention_diff_mma");
        return out;
    }
    // grids and scratch of a single-token step are sized for the longest sequence the cache allows, so that the launch is
    // the same at every step
    if (q.dtype == DType::BF16 && ctx.is_decode && illm_attention_diff_decode_supported(g.n_heads, g.n_kv_heads, g.head_dim, dv)) {
        const int group = g.n_heads / g.n_kv_heads, hb = group >= 8 ? 8 : group > 2 ? 4 : group;
        const int splits = attention_diff_splits(q.rows, g.n_kv_heads * (int)ceil_div(group, hb), ctx.max_seq_len, dev.n_sms());
        float* scratch = dev.alloc_n<float>((size_t)illm_attention_diff_scratch((int)q.rows, g.n_heads, dv, splits));
        check_kernel(illm_attention_diff_decode(q.p, (int)q.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p, (int)q.rows, g.n_heads,
                                                g.n_kv_heads, g.head_dim, dv, kv.page_size, kv.window, scale, p.lambda, p.eps, p.out_scale, ctx.max_seq_len,
                                                splits, scratch, dev.stream()),
                     "attention_diff_decode");
        return out;
    }
    check_kernel(illm_attention_diff(q.p, (int)q.cols, kv.k, kv.v, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p, code_of(q.dtype, "attention_diff"),
                                     (int)q.rows, g.n_heads, g.n_kv_heads, g.head_dim, dv, kv.page_size, kv.window, scale, p.lambda, p.eps, p.out_scale,
                                     1, nullptr, dev.stream()),
                 "attention_diff");
    return out;
}

int attention_diff_splits(long long T, int head_groups, long long max_seq_len, int n_sms) {
    const long long pairs = std::max<long long>(1, T * head_groups);
    long long s = std::max<long long>(1, 2LL * n_sms / pairs);
    s = std::min<long long>(s, std::max<long long>(1, ceil_div(max_seq_len, 256)));
    return (int)std::max<long long>(1, std::min<long long>(s, 64));
}

Mat attention(Device& dev, const Mat& qkv, const KVView& kv, const StepView& ctx, Geometry g, float scale) {
    const int nh = g.n_heads, nkv = g.n_kv_heads, d = g.head_dim, group = nkv ? nh / nkv : 0;
    // grids and scratch of the decode kernels are sized for the longest sequence the cache allows, so
    // that the launch is the same at every step
    if (ctx.is_decode && attention_decode_ring_supported(qkv.dtype, nh, nkv, d, kv.page_size)) {
        MatOrPartials in;
        in.m = qkv;
        return attention_decode_ring(dev, in, kv, ctx, g, scale, ctx.max_seq_len, 0, nullptr);
    }
    if (ctx.is_decode && (group >= kGqaDecodeMinGroup || !attention_decode_supported(qkv.dtype, nh, nkv, d, kv.page_size)) &&
        attention_decode_gqa_supported(qkv.dtype, nh, nkv, d))
        return attention_decode_gqa(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len);
    if (ctx.is_decode && attention_decode_supported(qkv.dtype, nh, nkv, d, kv.page_size))
        return attention_decode(dev, qkv, kv, ctx, g, scale, ctx.max_seq_len);
    if (!ctx.is_decode && attention_prefill_tc_supported(qkv.dtype, nh, nkv, d, kv.page_size))
        return attention_prefill_tc(dev, qkv, kv, ctx, g, scale);
    if (!ctx.is_decode && attention_prefill_supported(qkv.dtype, nh, nkv, d)) return attention_prefill(dev, qkv, kv, ctx, g, scale);
    return attention_generic(dev, qkv, kv, ctx, g, scale);
}

// ---- pieces of further mixers, feed-forwards and embeddings

int gate_act_from_name(const std::string& name) {
    if (name == "silu") return kActSilu;
    if (name == "relu") return kActRelu;
    if (name == "gelu_tanh") return kActGeluTanh;
    if (name == "swish_clamped") return kActSwishClamped;
    return -1;
}

Mat add2_rmsnorm(Device& dev, const Mat& resid, const Mat& d1, const Mat* d2, const Mat& w, float eps, DType out_dtype) {
    need(resid, "resid", true, DType::F32);
    need(d1, "delta", true, DType::F32);
    need(w, "norm weight", true, DType::F32);
    if (d2) need(*d2, "second delta", true, DType::F32);
    if (d1.rows != resid.rows || d1.cols != resid.cols || (d2 && (d2->rows != resid.rows || d2->cols != resid.cols)) || w.rows * w.cols != resid.cols)
        throw KernelError("add2_rmsnorm: the additions and the weight must have the stream's shape");
    if (resid.cols > kMaxNormWidth) throw KernelError("add2_rmsnorm: width " + std::to_string(resid.cols) + " exceeds what one block's shared memory holds");
    Mat y = new_mat(dev, resid.rows, resid.cols, out_dtype);
    check_kernel(illm_add2_rmsnorm((float*)resid.p, (const float*)d1.p, d2 ? (const float*)d2->p : nullptr, (const float*)w.p, y.p,
                                   code_of(out_dtype, "add2_rmsnorm"), (int)resid.rows, (int)resid.cols, eps, dev.stream()),
                 "add2_rmsnorm");
    return y;
}

Mat scaled_add_rmsnorm(Device& dev, const Mat& resid, const Mat& delta, const float* ls, const Mat* w, float eps, DType out_dtype) {
    need(resid, "resid", true, DType::F32);
    need(delta, "delta", true, DType::F32);
    if (w) need(*w, "norm weight", true, DType::F32);
    if (!ls) throw KernelError("scaled_add_rmsnorm: no layer scale");
    if (delta.rows != resid.rows || delta.cols != resid.cols || (w && w->rows * w->cols != resid.cols))
        throw KernelError("scaled_add_rmsnorm: the addition and the weight must have the stream's shape");
    if (resid.cols > kMaxNormWidth) throw KernelError("scaled_add_rmsnorm: width " + std::to_string(resid.cols) + " exceeds what one block's shared memory holds");
    Mat y;
    if (w) y = new_mat(dev, resid.rows, resid.cols, out_dtype);
    check_kernel(illm_scaled_add_rmsnorm((float*)resid.p, (const float*)delta.p, ls, w ? (const float*)w->p : nullptr, y.p,
                                         code_of(out_dtype, "scaled_add_rmsnorm"), (int)resid.rows, (int)resid.cols, eps, dev.stream()),
                 "scaled_add_rmsnorm");
    return y;
}

void add_bias(Device& dev, const Mat& y, const float* bias) {
    need(y, "y");
    if (!bias) throw KernelError("add_bias: no bias");
    check_kernel(illm_add_bias(y.p, code_of(y.dtype, "add_bias"), bias, (int)y.rows, (int)y.cols, dev.stream()), "add_bias");
}

Mat take_columns(Device& dev, const Mat& x, long long off, long long n, DType dtype) {
    need(x, "x", true, DType::F32);
    if (off < 0 || n <= 0 || off + n > x.cols) throw KernelError("take_columns: the columns lie outside the matrix");
    Mat y = new_mat(dev, x.rows, n, dtype);
    check_kernel(illm_take_columns((const float*)x.p, (int)x.cols, (int)off, (int)n, y.p, code_of(dtype, "take_columns"), (int)x.rows, dev.stream()),
                 "take_columns");
    return y;
}

Mat join_rows(Device& dev, const Mat& a, const Mat& b, DType dtype) {
    need(a, "a", true, DType::F32);
    need(b, "b", true, DType::F32);
    if (a.rows != b.rows || a.cols != b.cols) throw KernelError("join_rows: the two matrices differ in shape");
    Mat y = new_mat(dev, a.rows, 2 * a.cols, dtype);
    check_kernel(illm_join_rows((const float*)a.p, (const float*)b.p, (int)a.cols, y.p, code_of(dtype, "join_rows"), (int)a.rows, dev.stream()),
                 "join_rows");
    return y;
}

Mat bigram_embedding(Device& dev, const StepView& ctx, const Mat& table, const Mat& bigram, const BigramHash& hash, const StateView& last) {
    need(table, "table");
    need(bigram, "bigram table");
    if (bigram.dtype != table.dtype || bigram.cols != table.cols || bigram.rows != hash.buckets + 1)
        throw KernelError("bigram_embedding: the bigram table must have buckets + 1 rows of the embedding's width and dtype");
    if (!last.state || last.dtype != DType::I32 || last.elements < 1) throw KernelError("bigram_embedding: the state entry must hold one int32 per sequence");
    if (last.elements != 1) throw KernelError("bigram_embedding: the state entry must hold exactly one int32 per sequence");
    Mat out = new_mat_exact(dev, ctx.T, table.cols, DType::F32);
    check_kernel(illm_bigram_embedding(ctx.ids, ctx.token_pos, ctx.token_seq, ctx.cu_q, last.slots, (int*)last.state, table.p, bigram.p,
                                       code_of(table.dtype, "bigram_embedding"), (float*)out.p, ctx.T, ctx.B, (int)table.cols, (int)table.rows,
                                       (int)hash.buckets, hash.mul_prev, hash.mul_cur, ctx.err, dev.stream()),
                 "bigram_embedding");
    return out;
}

long long delta_rule_state_elements(int nh, int nkv, int d, int dv, int taps) {
    return (long long)nh * d * dv + (long long)(taps - 1) * (2LL * nkv * d + (long long)nh * dv);
}
bool delta_rule_supported(int d, int dv, int taps) { return illm_delta_rule_supported(d, dv, taps) != 0; }

Mat delta_rule(Device& dev, const Mat& x, const Mat& a, const DeltaRule& p, const StepView& ctx, const StateView& st) {
    need(x, "the packed projection", true, DType::F32);
    need(a, "the decay projection", true, DType::F32);
    const long long T = x.rows, C = 2LL * p.n_kv_heads * p.head_dim + (long long)p.n_heads * p.v_head_dim;
    if (a.rows != T || a.cols != (long long)p.n_heads * p.head_dim) throw KernelError("delta_rule: the decay projection must be [T, heads * head_dim]");
    if (!st.state || st.dtype != DType::F32 || st.elements != delta_rule_state_elements(p.n_heads, p.n_kv_heads, p.head_dim, p.v_head_dim, p.taps))
        throw KernelError("delta_rule: the state entry does not have this layer's size");
    Mat qkv = new_mat_exact(dev, T, C, DType::F32), g = new_mat_exact(dev, T, a.cols, DType::F32), beta = new_mat_exact(dev, T, p.n_heads, DType::F32);
    Mat out = new_mat_exact(dev, T, (long long)p.n_heads * p.v_head_dim, DType::F32);
    check_kernel(illm_delta_rule((const float*)x.p, (int)T, (int)x.cols, p.q_off, p.k_off, p.v_off, p.b_off, (const float*)a.p, p.n_heads,
                                 p.n_kv_heads, p.head_dim, p.v_head_dim, p.taps, p.conv_q, p.conv_k, p.conv_v, p.a_log, p.dt_bias, p.q_scale,
                                 (float*)st.state, st.elements, st.slots, ctx.cu_q, ctx.token_pos, ctx.token_seq, ctx.seq_lens, (float*)qkv.p,
                                 (float*)g.p, (float*)beta.p, (float*)out.p, ctx.B, dev.stream()),
                 "delta_rule");
    return out;
}

Mat latent_prep(Device& dev, const Mat& x, int q_rank, int kv_rank, const float* w_q, const float* w_kv, float eps, const StepView& ctx,
                const KVView& kv, DType act_dtype) {
    need(x, "the packed latent projection", true, DType::F32);
    if (x.cols < q_rank + kv_rank) throw KernelError("latent_prep: the projection is narrower than the two latents");
    if (kv.writes) {
        if (!kv.k || kv.dtype != act_dtype || kv.n_kv_heads != 1 || kv.head_dim != kv_rank)
            throw KernelError("latent_prep: the cache entry must hold one head of kv_rank channels in the activation dtype");
    }
    Mat cq = new_mat(dev, x.rows, q_rank, act_dtype);
    check_kernel(illm_latent_prep((const float*)x.p, (int)x.cols, q_rank, kv_rank, w_q, w_kv, eps, ctx.token_pos, ctx.token_seq, kv.block_table,
                                  kv.width, kv.page_size, cq.p, kv.writes ? kv.k : nullptr, code_of(act_dtype, "latent_prep"), (int)x.rows,
                                  ctx.err, dev.stream()),
                 "latent_prep");
    return cq;
}

Mat latent_attention_any(Device& dev, const Mat& q, const KVView& kv, const StepView& ctx, int heads, float scale, const float* gate, int gate_stride) {
    need(q, "q");
    if (!kv.k || kv.n_kv_heads != 1 || kv.dtype != q.dtype || q.cols != (long long)heads * kv.head_dim)
        throw KernelError("latent_attention_any: the queries and the cache entry (one head, the queries' dtype) do not fit together");
    Mat out = new_mat(dev, q.rows, q.cols, q.dtype);
    const int rc = illm_latent_attention_any_gated(q.p, kv.k, kv.block_table, kv.width, ctx.token_pos, ctx.token_seq, out.p, code_of(q.dtype, "latent_attention_any"),
                                                   (int)q.rows, heads, kv.head_dim, kv.page_size, kv.window, scale, gate, gate_stride, dev.stream());
    if (rc == 10001) throw KernelError("latent_attention_any: a latent of " + std::to_string(kv.head_dim) + " channels is beyond the kernel (up to 1024)");
    check_kernel(rc, "latent_attention_any");
    return out;
}

Mat head_linear(Device& dev, const Mat& x, const Mat& w, int heads, bool transposed, DType out_dtype) {
    return head_linear_pieces(dev, x, w, heads, transposed, out_dtype, HeadPieces());
}

Mat head_linear_pieces(Device& dev, const Mat& x, const Mat& w, int heads, bool transposed, DType out_dtype, const HeadPieces& pc) {
    need(x, "x");
    need(w, "w");
    if (heads <= 0 || x.cols % heads) throw KernelError("head_linear: the input's width is not a multiple of the head count");
    const long long x_hs = x.cols / heads;
    if (pc.x_head_stride && pc.x_head_stride != x_hs) throw KernelError("head_linear: the input's width is not heads x the given piece");
    long long K, N;
    if (transposed) {
        if (w.rows % heads) throw KernelError("head_linear: the matrix must have heads * n_in rows");
        K = w.rows / heads;
        N = w.cols;
    } else {
        if (w.rows % heads) throw KernelError("head_linear: the matrix must be [heads * n_out, n_in]");
        K = w.cols;
        N = w.rows / heads;
    }
    if (K > x_hs || (!pc.x_head_stride && K != x_hs)) throw KernelError("head_linear: the matrix does not fit the input's heads");
    Mat y;
    long long y_hs = N;
    if (pc.into) {
        y = *pc.into;
        y_hs = pc.y_head_stride;
        if (!y.p || y.dtype != out_dtype || y.rows != x.rows || y_hs < N || y.cols != heads * y_hs)
            throw KernelError("head_linear: the matrix to write into must be [T, heads x its piece] of the output dtype");
    } else {
        y = new_mat(dev, x.rows, (long long)heads * N, out_dtype);
    }
    // prompts in bfloat16: the library's batched product (a head per batch entry); few rows and float32: the kernel here
    if (x.dtype == DType::BF16 && w.dtype == DType::BF16 && out_dtype == DType::BF16 && x.rows > kGemmTcMaxTokensAuto && K % 8 == 0 && N % 8 == 0 &&
        x_hs % 8 == 0 && y_hs % 8 == 0 && !((uintptr_t)x.p & 15) && !((uintptr_t)w.p & 15) && !((uintptr_t)y.p & 15)) {
        dev.library_gemm_bf16_heads(x.p, w.p, y.p, (int)x.rows, (int)N, (int)K, heads, transposed, (int)x.cols, x_hs, (int)y.cols, y_hs);
        return y;
    }
    const int rc = illm_head_gemm_ex(x.p, code_of(x.dtype, "head_linear"), w.p, code_of(w.dtype, "head_linear"), y.p, code_of(out_dtype, "head_linear"),
                                     (int)x.rows, heads, (int)N, (int)K, transposed ? 1 : 0, (int)x.cols, (int)x_hs, (int)y.cols, (int)y_hs, dev.stream());
    if (rc == 10001) throw KernelError("head_linear: this combination of dtypes and sizes is not supported");
    check_kernel(rc, "head_linear");
    return y;
}

Mat latent_rope_prep(Device& dev, const Mat& x, const LatentRope& p, const StepView& ctx, const KVView& kv, DType act_dtype, Mat* qa) {
    need(x, "the packed latent projection", true, DType::F32);
    const long long row = (long long)p.kv_rank + p.rot_head_dim;
    if (p.n_heads <= 0 || p.head_dim <= 0 || p.rot_head_dim < 0 || p.kv_rank <= 0 || p.q_off < 0 || p.c_off < 0 ||
        p.q_off + (long long)p.n_heads * (p.head_dim + p.rot_head_dim) > x.cols || p.c_off + row > x.cols)
        throw KernelError("latent_rope_prep: the projection is narrower than the queries and the latent");
    if (p.rot_dim && !p.cos_sin) throw KernelError("latent_rope_prep: a rotation needs its cos/sin table");
    if (kv.writes && (!kv.k || kv.dtype != act_dtype || kv.n_kv_heads != 1 || kv.head_dim != row))
        throw KernelError("latent_rope_prep: the cache entry must hold one head of kv_rank + rotated channels in the activation dtype");
    if (!qa) throw KernelError("latent_rope_prep: nowhere to put the absorbed queries");
    *qa = new_mat(dev, x.rows, p.n_heads * row, act_dtype);
    const bool q_f32 = ctx.is_decode || act_dtype == DType::F32;
    Mat qn = new_mat(dev, x.rows, (long long)p.n_heads * p.head_dim, q_f32 ? DType::F32 : act_dtype);
    check_kernel(illm_latent_rope_prep((const float*)x.p, (int)x.cols, p.q_off, p.n_heads, p.head_dim, p.rot_head_dim, p.c_off, p.kv_rank, p.w_kv, p.eps,
                                       p.cos_sin, p.rot_dim, p.pairs ? 1 : 0, (int)p.n_pos, ctx.token_pos, ctx.token_seq, kv.block_table, kv.width,
                                       kv.page_size, qn.p, q_f32 ? 1 : 0, qa->p, kv.writes ? kv.k : nullptr, code_of(act_dtype, "latent_rope_prep"),
                                       (int)x.rows, ctx.err, dev.stream()),
                 "latent_rope_prep");
    return qn;
}

Mat moe_forward(Device& dev, const Mat& h, const Mat& logits, const float* router_bias, int E, int top, const Mat& w_gu, const Mat& w_down, int act) {
    MoeRouting r;
    r.bias = router_bias;
    return moe_forward_ex(dev, h, logits, r, E, top, w_gu, w_down, act);
}

Mat moe_forward_ex(Device& dev, const Mat& h, const Mat& logits, const MoeRouting& r, int E, int top, const Mat& w_gu, const Mat& w_down, int act) {
    need(h, "h");
    need(logits, "the router's logits", true, DType::F32);
    const long long T = h.rows, D = h.cols;
    if (logits.rows != T || logits.cols != E || top <= 0 || top > E) throw KernelError("moe: the router's logits must be [T, experts] and top within the experts");
    if (w_gu.dtype != h.dtype || w_down.dtype != h.dtype || w_gu.cols != D || w_gu.rows % (2 * E) || w_down.cols * 2 * E != w_gu.rows ||
        w_down.rows != (long long)E * D)
        throw KernelError("moe: the experts' matrices do not match the input");
    const long long F = w_down.cols, P = T * top;
    // bfloat16 with rows of whole 16-byte pieces runs on tensor cores: prompts on tcgen05 (tiles of 128 rows of the rows
    // gathered into the experts' order), few rows on warp-level MMA; float32 (and odd sizes) on the plain kernel
    const int tc = h.dtype == DType::BF16 && D % 8 == 0 && F % 8 == 0 ? 1 : 0;
    const bool tc5 = tc && P >= kMoeTcgen05MinRows;
    const int bm = tc5 ? 128 : illm_moe_row_tile((int)T, top, tc);
    const int tiles = illm_moe_max_tiles((int)T, top, E, bm);
    int* expert = dev.alloc_n<int>((size_t)P);
    float* weight = dev.alloc_n<float>((size_t)P);
    int* row_of_pair = dev.alloc_n<int>((size_t)P);
    int* pair_of_row = dev.alloc_n<int>((size_t)P);
    int* tile_expert = dev.alloc_n<int>((size_t)tiles);
    int* tile_row0 = dev.alloc_n<int>((size_t)tiles);
    int* tile_rows = dev.alloc_n<int>((size_t)tiles);
    if (r.scoring >= 1 && (r.groups < 1 || r.groups > 32 || E % r.groups || r.keep < 1 || r.keep > r.groups || (long long)r.keep * (E / r.groups) < top))
        throw KernelError("moe: the experts must form up to 32 equal groups, and the groups kept must hold at least `top` experts");
    if (r.plus && (r.plus->dtype != DType::F32 || r.plus->rows != T || r.plus->cols != D)) throw KernelError("moe: the addend must be float32 [T, hidden]");
    if (r.scoring < 0 || r.scoring > 2 || r.group_top < 1 || r.group_top > 4) throw KernelError("moe: unknown scoring, or a group score of more than 4 experts");
    if (act == kActSwishClamped && !(r.act_limit > 0.f)) throw KernelError("moe: the clamped activation needs a positive limit");
    check_kernel(illm_moe_route_ex2((const float*)logits.p, r.bias, (int)T, E, top, bm, r.scoring, r.groups, r.keep, r.renorm ? 1 : 0, r.group_top, r.sum_eps,
                                    r.weight_scale, expert, weight, row_of_pair, pair_of_row, tile_expert, tile_row0, tile_rows, dev.stream()),
                 "moe_route");
    const int code = code_of(h.dtype, "moe");
    Mat hid = new_mat_exact(dev, P, F, h.dtype), rows = new_mat_exact(dev, P, D, DType::F32), out = new_mat_exact(dev, T, D, DType::F32);
    if (tc5) {
        Mat xs = new_mat_exact(dev, P, D, DType::BF16);
        check_kernel(illm_moe_gather_rows(h.p, xs.p, pair_of_row, (int)P, (int)D, top, dev.stream()), "moe_gather_rows");
        check_kernel(illm_moe_gemm_tc_ex(xs.p, w_gu.p, hid.p, (int)P, E, (int)(2 * F), (int)D, 1, act, r.act_limit, tiles, tile_expert, tile_row0, tile_rows,
                                      dev.tc_error_word(), dev.stream()),
                     "moe_gemm_tc (gate/up)");
        check_kernel(illm_moe_gemm_tc(hid.p, w_down.p, rows.p, (int)P, E, (int)D, (int)F, 0, 0, tiles, tile_expert, tile_row0, tile_rows,
                                      dev.tc_error_word(), dev.stream()),
                     "moe_gemm_tc (down)");
    } else {
        check_kernel(illm_moe_gemm_ex(h.p, code, w_gu.p, code, hid.p, (int)T, top, E, (int)(2 * F), (int)D, 1, act, r.act_limit, bm, tc, pair_of_row, tile_expert, tile_row0,
                                   tile_rows, dev.stream()),
                     "moe_gemm (gate/up)");
        check_kernel(illm_moe_gemm(hid.p, code, w_down.p, code, rows.p, (int)T, top, E, (int)D, (int)F, 0, 0, bm, tc, pair_of_row, tile_expert, tile_row0,
                                   tile_rows, dev.stream()),
                     "moe_gemm (down)");
    }
    check_kernel(illm_moe_combine_plus((const float*)rows.p, row_of_pair, weight, r.plus ? (const float*)r.plus->p : nullptr, (float*)out.p, (int)T, (int)D, top,
                                       dev.stream()),
                 "moe_combine");
    return out;
}

// ---- sampling and utilities

int* argmax(Device& dev, const float* logits, long long B, long long V, int* out) {
    if (!out) out = dev.alloc_n<int>((size_t)std::max<long long>(B, 1));
    const long long n_chunks = ceil_div(V, 2048);
    for (long long b0 = 0; b0 < B; b0 += 65535) {
        const long long b1 = std::min(B, b0 + 65535);
        float* sv = dev.alloc_n<float>((size_t)(b1 - b0) * n_chunks);
        int* si = dev.alloc_n<int>((size_t)(b1 - b0) * n_chunks);
        check_kernel(illm_argmax(logits + (size_t)b0 * V, (int)(b1 - b0), (int)V, (int)V, out + b0, sv, si, dev.stream()), "argmax");
    }
    return out;
}

int* sample(Device& dev, const float* logits, long long B, long long V, const float* uniforms, float temp, int top_k, float top_p,
            float repeat_penalty, const int* last_tokens, int n_last, int* out) {
    if (!out) out = dev.alloc_n<int>((size_t)std::max<long long>(B, 1));
    float* z = dev.alloc_n<float>((size_t)B * V);
    for (long long b0 = 0; b0 < B; b0 += 65535) {
        const long long b1 = std::min(B, b0 + 65535);
        // temperature alone and top_k <= 64 run in two passes over chunks of the row and need scratch
        const long long n_scratch = illm_sample_scratch_elems((int)(b1 - b0), (int)V, top_k, top_p);
        int* scratch = n_scratch ? dev.alloc_n<int>((size_t)n_scratch) : nullptr;
        check_kernel(illm_sample(logits + (size_t)b0 * V, (int)(b1 - b0), (int)V, (int)V, z + (size_t)b0 * V,
                                 last_tokens ? last_tokens + (size_t)b0 * n_last : nullptr, last_tokens ? n_last : 0, temp, repeat_penalty, top_k,
                                 top_p, uniforms + b0, out + b0, scratch, dev.stream()),
                     "sample");
    }
    return out;
}

void fill_random(Device& dev, void* out, DType dtype, long long n, unsigned long long key, float std, float mean) {
    check_kernel(illm_fill_random(out, code_of(dtype, "fill_random"), n, key, std, mean, dev.stream()), "fill_random");
}

void convert(Device& dev, const void* src, DType src_dtype, void* dst, DType dst_dtype, long long n) {
    const int rc = illm_convert(src, (int)src_dtype, dst, (int)dst_dtype, n, dev.stream());
    if (rc == 10001)
        throw KernelError(std::string("a tensor stored as ") + dtype_word(src_dtype) + " cannot be brought to " + dtype_word(dst_dtype));
    check_kernel(rc, "convert");
}

Mat cast(Device& dev, const Mat& x, DType dtype) {
    if (x.dtype == dtype) return x;
    Mat y = new_mat(dev, x.rows, x.cols, dtype);
    convert(dev, x.p, x.dtype, y.p, dtype, x.rows * x.cols);
    return y;
}

}  // namespace ops
}  // namespace illm
