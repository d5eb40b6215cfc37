#include "ops.h"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <tuple>

#include "kernels.h"

namespace sandy {
namespace ops {

namespace {

int code_of(DType d) {
    if (d == DType::F32) return 0;
    if (d == DType::BF16) return 1;
    throw UnsupportedShape("kernels take float32 or bfloat16 tensors");
}

void check(int code, const std::string& what) {
    g_launches++;
    if (code == 0) return;
    if (code == -1) throw UnsupportedShape(what + ": sizes or dtypes not supported by this kernel");
    if (code == -2) throw KernelError(what + ": bad argument (null pointer or impossible size)");
    throw KernelError(what + ": CUDA error " + std::to_string(code) + " (" + cudaGetErrorString((cudaError_t)code) + ")");
}

bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) return false;
    return st != cudaStreamCaptureStatusNone;
}

int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : fallback;
}

// ---- per-class timing ---------------------------------------------------------------------------
struct OpRecord {
    const char* op_class;
    cudaEvent_t e0, e1;
    double bytes, flops;
};
bool g_profile = false;
std::vector<OpRecord> g_records;

class OpTimer {
public:
    OpTimer(const Launch& l, const char* op_class, double bytes, double flops) : stream_(l.stream) {
        if (!g_profile || capturing(l.stream)) return;
        rec_.op_class = op_class;
        rec_.bytes = bytes;
        rec_.flops = flops;
        if (cudaEventCreate(&rec_.e0) != cudaSuccess || cudaEventCreate(&rec_.e1) != cudaSuccess) return;
        cudaEventRecord(rec_.e0, stream_);
        on_ = true;
    }
    ~OpTimer() {
        if (!on_) return;
        cudaEventRecord(rec_.e1, stream_);
        g_records.push_back(rec_);
    }
private:
    cudaStream_t stream_;
    OpRecord rec_{};
    bool on_ = false;
};

// ---- leaving launches out -------------------------------------------------------------------------
// What a kernel costs inside a step -- where its set-up runs under the tail of the kernel before and the
// next one's under its own -- is not what it takes when timed alone.  For that figure a step is timed with
// a family of launches left out (its results are then garbage; only the time is read) and the difference
// to the whole step taken: families "layernorm", "attention", "kv_append", and "product" or
// "product <N>x<K>" for the products of one shape.  Set through the control plane (leave_out); graphs
// recorded before a change still hold the launches, so a fresh engine is made for every setting.
std::vector<std::string> g_left_out;

bool left_out(const char* family, int64_t N = 0, int64_t K = 0) {
    if (g_left_out.empty()) return false;
    const std::string f = family;
    const std::string shaped = N ? f + " " + std::to_string(N) + "x" + std::to_string(K) : f;
    for (const std::string& x : g_left_out)
        if (x == f || x == shaped) return true;
    return false;
}

double tensor_bytes(const Tensor* t) { return t ? (double)t->numel() * (double)t->elem_size() : 0.0; }

std::string dims(const Tensor& t) { return "[" + std::to_string(t.rows) + ", " + std::to_string(t.cols) + "]"; }

}  // namespace

Act act_from_name(const std::string& name) {
    if (name.empty() || name == "none") return Act::None;
    if (name == "gelu_new" || name == "gelu_tanh") return Act::GeluNew;
    if (name == "gelu" || name == "gelu_erf") return Act::Gelu;
    if (name == "relu_squared") return Act::ReluSquared;
    throw ValueError("unknown activation '" + name + "'");
}

const char* kernel_status_text() {
    return "bits 0-2 a barrier wait ran out in the tensor-core product, bit 3 a key/value write and bit 4 a key read had "
           "no page behind it, bits 5-6 a wait ran out in the bulk decode attention, bit 8 in the tcgen05 prefill attention";
}

void profile_enable(bool on) { g_profile = on; }

void leave_out(const std::vector<std::string>& families) { g_left_out = families; }

std::vector<ProfileRow> profile_report() {
    std::map<std::string, ProfileRow> by_class;
    for (OpRecord& r : g_records) {
        float ms = 0;
        if (cudaEventSynchronize(r.e1) == cudaSuccess) cudaEventElapsedTime(&ms, r.e0, r.e1);
        ProfileRow& row = by_class[r.op_class];
        row.op_class = r.op_class;
        row.calls++;
        row.us += 1e3 * ms;
        row.bytes += r.bytes;
        row.flops += r.flops;
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    g_records.clear();
    std::vector<ProfileRow> out;
    for (auto& kv : by_class) out.push_back(kv.second);
    return out;
}

int sm_count() {
    static int n = 0;
    if (n == 0) n = SANDY_KERNEL(embed, sandy_device_sm_count)();
    return n;
}

void spin(cudaStream_t stream, long long nanoseconds) {
    static auto fn = SANDY_KERNEL(embed, sandy_spin);
    const int code = fn(nanoseconds, stream);
    if (code) throw KernelError("spin: CUDA error " + std::to_string(code));
}

void embed_positions(const Launch& l, const int* ids, const int* positions, const Tensor& wte, const Tensor* wpe, Tensor& out,
                     int n_tokens) {
    if (wpe && (wpe->dtype != wte.dtype || wpe->cols != out.cols))
        throw KernelError("position table must match the token table in dtype and width");
    if (wte.cols != out.cols || !wte.contiguous() || !out.contiguous() || out.rows < n_tokens)
        throw KernelError("embed_positions: tables and output must be contiguous and of one width");
    static auto fn = SANDY_KERNEL(embed, sandy_embed_pos);
    OpTimer timer(l, "embedding", (double)n_tokens * out.cols * ((wpe ? 2.0 : 1.0) * wte.elem_size() + out.elem_size()), 0);
    check(fn(ids, positions, wte.data, wpe ? wpe->data : nullptr, out.data, n_tokens, (int)out.cols, (int)wte.rows,
             wpe ? (int)wpe->rows : 0, code_of(wte.dtype), code_of(out.dtype), l.status, l.stream),
          "embed_positions");
}

void layernorm(const Launch& l, const Tensor& x, const Tensor& gamma, const Tensor* beta, float eps, Tensor& out,
               const int* rows, int n_rows) {
    const int64_t width = x.cols;
    if (!rows && x.rows < n_rows) throw KernelError("layernorm: x and out disagree");
    if (!x.contiguous() || !out.contiguous() || out.cols != width || gamma.numel() != width || out.rows < n_rows)
        throw KernelError("layernorm: contiguous [rows, width] tensors expected");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(norm, sandy_layernorm);
    OpTimer timer(l, "layernorm", (double)n_rows * width * (x.elem_size() + out.elem_size()), 0);
    check(fn(x.data, gamma.data, beta ? beta->data : nullptr, out.data, rows, n_rows, (int)width, eps, code_of(x.dtype),
             code_of(gamma.dtype), code_of(out.dtype), l.stream),
          "layernorm(width=" + std::to_string(width) + ")");
}

void gemm_simt(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, bool w_out_in, Act act,
               const Tensor* residual) {
    const int64_t M = a.rows, K = a.cols, N = out.cols;
    const int64_t wk = w_out_in ? w.cols : w.rows, wn = w_out_in ? w.rows : w.cols;
    if (wk != K || wn != N || out.rows != M)
        throw KernelError("gemm: shapes disagree: a " + dims(a) + ", w " + dims(w) + (w_out_in ? " (out_in)" : " (in_out)") +
                          ", out " + dims(out));
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm: residual must be float32 [M, N]");
    if (bias && (bias->dtype != w.dtype || bias->numel() != N)) throw KernelError("gemm: bias must have the weight's dtype and N elements");
    static auto fn = SANDY_KERNEL(gemm_simt, sandy_gemm_simt);
    OpTimer timer(l, "product, FFMA (float32)", tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual),
                  2.0 * M * N * K);
    check(fn(a.data, w.data, bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M,
             (int)N, (int)K, (int)a.ld, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, w_out_in ? 1 : 0, (int)act,
             code_of(a.dtype), code_of(w.dtype), code_of(out.dtype), l.stream),
          "gemm_simt(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
}

bool tensor_core_gemm_supported(int64_t K, int64_t N) {
    (void)N;
    return K % 8 == 0 && K >= 8;       // operand rows must start on 16-byte boundaries for TMA
}

// ---- the tcgen05 product and its variants -----------------------------------------------------------
// Which of the tcgen05 variants (three tile widths, one tile per CTA or persistent; two CTAs on a
// 256-row tile, two widths) is fastest depends on how the tiles of a product fall on the SMs, and a
// model of it was off by 20 % on half the shapes tried.  So the first product of a shape (rows in
// steps of 128) with at least 256 rows times each variant on a scratch output and remembers the
// winner.  All variants add the k-steps of an output element in the same order, so the choice never
// changes a result.  Not done while a CUDA graph is being captured (the kernel's own default stands
// then).  Tile codes: n < 0 one tile of 128 x |n| per CTA, n > 0 the persistent kernel with tiles of
// 128 x n, kPairTile + n two CTAs on a 256 x n tile.
constexpr int kPairTile = 2000;
constexpr int kGemmTuneMinRows = 256;
constexpr int kTuneLaunches = 8;
const int kGemmVariants[] = {-64, -128, -256, 64, 128, 256, kPairTile + 128, kPairTile + 256};

namespace {
using TileKey = std::tuple<int64_t, int64_t, int64_t, int, bool, int>;
std::map<TileKey, int> g_tiles;
std::map<std::pair<int64_t, int64_t>, int> g_forced_tiles;      // (N, K) -> variant, for comparisons (force_tile)

struct TcArgs {
    const Tensor* a; const Tensor* w; const Tensor* bias; Act act; int64_t M, N, K;
};

void launch_tc(const Launch& l, const TcArgs& g, int tile, Tensor& dst, const Tensor* res, const KVTarget* kv) {
    static auto fn1 = SANDY_KERNEL(gemm_tc, sandy_gemm_tc);
    auto fn = fn1;
    if (tile >= kPairTile) {
        static auto fn2 = SANDY_KERNEL(gemm_tc2, sandy_gemm_tc2);
        fn = fn2;
        tile -= kPairTile;
    }
    const KVView* c = kv ? &kv->cache : nullptr;
    check(fn(g.a->data, g.w->data, g.bias ? g.bias->data : nullptr, res ? (const float*)res->data : nullptr, dst.data, (int)g.M,
             (int)g.N, (int)g.K, (int)g.a->ld, (int)g.w->ld, res ? (int)res->ld : 0, (int)dst.ld, (int)g.act, code_of(dst.dtype),
             tile, c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr,
             kv ? kv->max_blocks : 0, kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0,
             kv ? kv->kv_cols : 0, c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_tc(M=" + std::to_string(g.M) + ",N=" + std::to_string(g.N) + ",K=" + std::to_string(g.K) +
              ",tile=" + std::to_string(tile) + ")");
}
}  // namespace

void gemm_tc(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
             const Tensor* residual, int tile_n, KVTarget* kv) {
    const int64_t M = a.rows, K = a.cols, N = w.rows;
    if (a.dtype != DType::BF16 || w.dtype != DType::BF16) throw UnsupportedShape("gemm_tc takes bfloat16 operands");
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_tc: shapes disagree: a " + dims(a) + ", w " + dims(w) + ", out " + dims(out));
    if (K % 8 || a.ld % 8 || w.ld % 8 || ((uintptr_t)a.data & 15) || ((uintptr_t)w.data & 15))
        throw UnsupportedShape("gemm_tc: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_tc: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_tc: bias must be bfloat16 [N]");
    if (kv) {
        const KVView& c = kv->cache;
        if (c.dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c.n_kv_heads * c.head_dim ||
            kv->q_cols + 2 * kv->kv_cols != N)
            throw KernelError("gemm_tc: the key/value target does not match the product");
    }
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    OpTimer timer(l, kv ? "product, tcgen05 (+ cache write)" : "product, tcgen05",
                  tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual), 2.0 * M * N * K);
    const TcArgs g{&a, &w, bias, act, M, N, K};
    const TileKey key{(M + 127) / 128, N, K, (int)act, residual != nullptr, (int)out.dtype};
    if (tile_n == 0 && !g_forced_tiles.empty() && M >= kGemmTuneMinRows) {
        auto forced = g_forced_tiles.find({N, K});
        if (forced != g_forced_tiles.end()) tile_n = forced->second;
    }
    if (tile_n == 0) {
        auto hit = g_tiles.find(key);
        if (hit != g_tiles.end()) tile_n = hit->second;
        else if (M >= kGemmTuneMinRows && !capturing(l.stream)) {
            // timed without the cache write: the scratch runs must not touch pages.  A product that adds
            // into its own output (x += ...) is timed adding into the scratch, the way it will run.
            DeviceBuffer scratch((size_t)M * (size_t)N * out.elem_size());
            cuda_check(cudaMemsetAsync(scratch.get(), 0, (size_t)M * (size_t)N * out.elem_size(), l.stream), "clearing the tuner's scratch");
            Tensor dst = out;
            dst.data = scratch.get();
            dst.ld = N;
            const bool in_place = residual && residual->data == out.data;
            const Tensor* tune_res = in_place ? &dst : residual;
            cudaEvent_t e0, e1;
            cuda_check(cudaEventCreate(&e0), "creating an event");
            cuda_check(cudaEventCreate(&e1), "creating an event");
            float best_ms = 1e30f;
            int best = 0;
            static const bool tune_log = std::getenv("SANDYRT_TUNE_LOG") != nullptr;      // what the tuner saw, on stderr
            for (int tile : kGemmVariants) {
                launch_tc(l, g, tile, dst, tune_res, nullptr);
                // A launch costs the host about as long as one of these kernels takes the GPU, so timed
                // naively the host's pace is what is measured; here the GPU is kept busy with a spin kernel
                // while the launches queue up behind it.
                spin(l.stream, 300000);
                cudaEventRecord(e0, l.stream);
                for (int i = 0; i < kTuneLaunches; i++) launch_tc(l, g, tile, dst, tune_res, nullptr);
                cudaEventRecord(e1, l.stream);
                cuda_check(cudaEventSynchronize(e1), "timing a product");
                float ms = 0;
                cudaEventElapsedTime(&ms, e0, e1);
                if (ms < best_ms) { best_ms = ms; best = tile; }
                if (tune_log) fprintf(stderr, "[sandyrt_b200] product %lld x %lld x %lld, tile %d: %.2f us\n", (long long)M, (long long)N, (long long)K, tile, ms * 1e3f / kTuneLaunches);
            }
            if (tune_log) fprintf(stderr, "[sandyrt_b200] product %lld x %lld x %lld: tile %d\n", (long long)M, (long long)N, (long long)K, best);
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            g_tiles[key] = best;
            tile_n = best;
        }
    }
    launch_tc(l, g, tile_n, out, residual, kv);
    if (kv) kv->written = true;
}

// The variant that products of W [N, K] with at least 256 rows take from now on, whatever the tuner
// found (0: the tuner's choice again).  For comparing variants inside a whole step; steps already
// recorded as graphs keep what they were recorded with.
void force_tile(int64_t N, int64_t K, int tile) {
    if (tile == 0) g_forced_tiles.erase({N, K});
    else g_forced_tiles[{N, K}] = tile;
}

// ---- the weight-streaming product ---------------------------------------------------------------------
constexpr int kSkinnyNormMaxRows = 16;
constexpr int kSkinnyNormMaxK = 2048;
bool skinny_norm_fusable(const FusedNorm& n, int64_t K, DType out_dtype) {
    return n.gamma.dtype == DType::BF16 && out_dtype == DType::BF16 && n.x.dtype == DType::F32 &&
           n.x.rows <= kSkinnyNormMaxRows && K <= kSkinnyNormMaxK && n.x.ld % 4 == 0 && !((uintptr_t)n.x.data & 15) &&
           !((uintptr_t)n.gamma.data & 15) && (!n.beta || !((uintptr_t)n.beta->data & 15));
}

void gemm_skinny(const Launch& l, const Tensor* a, const FusedNorm* norm, const Tensor& w, const Tensor* bias, Tensor& out,
                 Act act, const Tensor* residual, KVTarget* kv) {
    const int64_t M = norm ? norm->x.rows : a->rows, K = norm ? norm->x.cols : a->cols, N = w.rows;
    if (norm && !skinny_norm_fusable(*norm, K, DType::BF16)) throw UnsupportedShape("gemm_skinny: this norm cannot be fused");
    if ((!norm && a->dtype != DType::BF16) || w.dtype != DType::BF16) throw UnsupportedShape("gemm_skinny takes bfloat16 operands");
    if (M > kSkinnyMaxRows) throw UnsupportedShape("gemm_skinny takes at most 64 rows, got " + std::to_string(M));
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_skinny: shapes disagree: a [" + std::to_string(M) + ", " + std::to_string(K) + "], w " + dims(w) +
                          ", out " + dims(out));
    if (K % 8 || w.ld % 8 || ((uintptr_t)w.data & 15) || (a && (a->ld % 8 || ((uintptr_t)a->data & 15))))
        throw UnsupportedShape("gemm_skinny: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_skinny: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_skinny: bias must be bfloat16 [N]");
    const KVView* c = kv ? &kv->cache : nullptr;
    if (kv && (c->dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c->n_kv_heads * c->head_dim ||
               kv->q_cols + 2 * kv->kv_cols != N))
        throw KernelError("gemm_skinny: the key/value target does not match the product");
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    static auto fn = SANDY_KERNEL(gemm_skinny, sandy_gemm_skinny);
    OpTimer timer(l, norm ? (kv ? "product, streaming (+ norm, cache write)" : "product, streaming (+ norm)") : "product, streaming",
                  (norm ? tensor_bytes(&norm->x) : tensor_bytes(a)) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual),
                  2.0 * M * N * K);
    check(fn(a ? a->data : nullptr, norm ? (const float*)norm->x.data : nullptr, norm ? (int)norm->x.ld : 0,
             norm ? norm->gamma.data : nullptr, (norm && norm->beta) ? norm->beta->data : nullptr, norm ? norm->eps : 0.0f, w.data,
             bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M, (int)N, (int)K,
             a ? (int)a->ld : 0, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, (int)act, code_of(out.dtype),
             c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr, kv ? kv->max_blocks : 0,
             kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0, kv ? kv->kv_cols : 0,
             c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_skinny(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
    if (kv) kv->written = true;
}

// ---- 17 to 64 rows on the tensor cores -----------------------------------------------------------------
// Which kernel a product of 17 to 64 rows gets.  Timed one kernel after itself the tcgen05 kernel with
// 64-wide tiles wins the up-projection (3072 x 768 at 64 rows: 6.8 us against 9.8 streaming) and split-K
// the down-projection (768 x 3072: 8.2 against 11.2) and the vocabulary (50257 x 768: 26 against 98).
// Inside a decode step of 64 requests, where a kernel's set-up and first loads run under the tail of the
// kernel before it if its blocks find room beside that kernel's, the streaming kernel with its small blocks
// beats the tiled one on the up-projection (step 0.723 ms against 0.756), split-K keeps its lead on the
// down-projection (0.756 against 0.820) and is level on the vocabulary.  So: split-K for a long K or very
// many columns, streaming otherwise.  The kernels add in different orders, so the choice is a fixed rule
// of the shape and never a timing: the same batch gives the same bfloat16 tokens in every process.
constexpr int kSmallMinRows = 17;
constexpr int kSplitKMinK = 2048;
constexpr int kSplitKMinCols = 16384;
// Below 17 rows the streaming kernel keeps the products up to K = 4,096 (8 rows, us alone, streaming / split-K:
// 768 x 3072 4.7 / 4.7 and a decode step 0.296 / 0.304 ms; 1024 x 4096 5.0 / 5.1; 1280 x 5120 8.1 / 6.2;
// 1600 x 6400 10.1 / 7.6).
constexpr int kSplitKMinKFewRows = 5120;
constexpr int kSplitKMinKManyRows = 1280;

SmallGemm small_gemm_kernel(int64_t M, int64_t N, int64_t K) {
    if (M < kSmallMinRows) return K >= kSplitKMinKFewRows ? SmallGemm::SplitK : SmallGemm::Skinny;
    if (K >= kSplitKMinK || N >= kSplitKMinCols) return SmallGemm::SplitK;
    // more than two row tiles of wide rows: the streaming kernel's blocks each fetch all rows (64 x 1,600: 205 KB)
    // (64 rows, us alone, streaming / split-K: 4800 x 1600 18.7 / 10.4, 1600 x 1600 10.0 / 7.7, 6400 x 1600 20.3 /
    // 14.5; at 32 rows level; at K = 1,024 the streaming kernel leads: 3072 x 1024 7.2 / 11.9)
    if (M > 32 && K >= kSplitKMinKManyRows) return SmallGemm::SplitK;
    return SmallGemm::Skinny;
}

void gemm_small(const Launch& l, const Tensor& a, const Tensor& w, const Tensor* bias, Tensor& out, Act act,
                const Tensor* residual, KVTarget* kv) {
    const int64_t M = a.rows, K = a.cols, N = w.rows;
    if (a.dtype != DType::BF16 || w.dtype != DType::BF16) throw UnsupportedShape("gemm_small takes bfloat16 operands");
    if (M > kSmallMaxRows) throw UnsupportedShape("gemm_small takes at most 256 rows, got " + std::to_string(M));
    if (w.cols != K || out.rows != M || out.cols != N)
        throw KernelError("gemm_small: shapes disagree: a " + dims(a) + ", w " + dims(w) + ", out " + dims(out));
    if (K % 8 || w.ld % 8 || a.ld % 8 || ((uintptr_t)w.data & 15) || ((uintptr_t)a.data & 15))
        throw UnsupportedShape("gemm_small: K=" + std::to_string(K) + " and the row pitches must be multiples of 8 elements, operands 16-byte aligned");
    if (residual && (residual->dtype != DType::F32 || residual->rows != M || residual->cols != N))
        throw KernelError("gemm_small: residual must be float32 [M, N]");
    if (bias && (bias->dtype != DType::BF16 || bias->numel() != N)) throw KernelError("gemm_small: bias must be bfloat16 [N]");
    const KVView* c = kv ? &kv->cache : nullptr;
    if (kv && (c->dtype != DType::BF16 || out.dtype != DType::BF16 || kv->kv_cols != c->n_kv_heads * c->head_dim ||
               kv->q_cols + 2 * kv->kv_cols != N))
        throw KernelError("gemm_small: the key/value target does not match the product");
    if (left_out("product", N, K)) {
        if (kv) kv->written = true;
        return;
    }
    static auto fn = SANDY_KERNEL(gemm_small, sandy_gemm_small);
    OpTimer timer(l, kv ? "product, tcgen05 split-K (+ cache write)" : "product, tcgen05 split-K",
                  tensor_bytes(&a) + tensor_bytes(&w) + tensor_bytes(&out) + 2 * tensor_bytes(residual), 2.0 * M * N * K);
    check(fn(a.data, w.data, bias ? bias->data : nullptr, residual ? (const float*)residual->data : nullptr, out.data, (int)M,
             (int)N, (int)K, (int)a.ld, (int)w.ld, residual ? (int)residual->ld : 0, (int)out.ld, (int)act, code_of(out.dtype),
             c ? c->k : nullptr, c ? c->v : nullptr, c ? c->page_stride : 0, kv ? kv->block_table : nullptr, kv ? kv->max_blocks : 0,
             kv ? kv->token_seq : nullptr, kv ? kv->positions : nullptr, kv ? kv->q_cols : 0, kv ? kv->kv_cols : 0,
             c ? c->head_dim : 0, c ? c->page_size : 0, c ? c->num_pages : 0, l.kernel_status, l.stream),
          "gemm_small(M=" + std::to_string(M) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
    if (kv) kv->written = true;
}

// ---- the cache and attention ------------------------------------------------------------------------------
void kv_append(const Launch& l, const Tensor& k_src, const Tensor& v_src, const KVView& c, const int* block_table,
               int max_blocks, const int* token_seq, const int* positions) {
    if (k_src.rows != v_src.rows || k_src.cols != v_src.cols || k_src.cols != (int64_t)c.n_kv_heads * c.head_dim ||
        k_src.ld != v_src.ld || k_src.dtype != c.dtype || v_src.dtype != c.dtype)
        throw KernelError("kv_append: sources must be [T, Hkv*D] of the cache's dtype with one stride");
    if (left_out("kv_append")) return;
    static auto fn = SANDY_KERNEL(attention, sandy_kv_append);
    OpTimer timer(l, "key/value append", 2 * (tensor_bytes(&k_src) + tensor_bytes(&v_src)), 0);
    check(fn(k_src.data, v_src.data, (int)k_src.ld, c.k, c.v, c.page_stride, block_table, max_blocks, token_seq, positions,
             (int)k_src.rows, c.n_kv_heads, c.head_dim, c.page_size, c.num_pages, code_of(c.dtype), l.kernel_status, l.stream),
          "kv_append");
}

int decode_splits(int n_tokens, int n_heads, int max_kv, int sms) {
    static const int forced = env_int("SANDYRT_DECODE_SPLITS", 0);       // > 0: this many splits, for comparisons
    if (forced > 0) return forced;
    if (sms <= 0) sms = sm_count();
    // About four blocks an SM in all, to the nearest number of splits.  (Rounded up, as it was for the
    // register kernel, 12 / 16 / 24 requests of 12 heads got 5 / 4 / 3 splits; whole decode steps with the
    // mma.sync kernel, GPT-2 small, context ~400, ms by splits 1 / 2 / 3 / 4 / 5: 12 requests .340 / .334 /
    // .323 / .311 / .342; 16: .361 / .350 / .341 / .361 / .374; 24: .490 / .409 / .455 / .437 / .473; 32:
    // .509 / .494 / .484 / .512 / .508; 48: .627 / .626 / .664 / .685 / .731; 8: .330 / .323 / .310 / .303 / .306.)
    // Long ranges: a block that walks more than some 256 keys alone is the step's longest chain, so a pair is
    // cut further as long as no more than eight blocks an SM come of it (32 requests at context 965, ms by
    // splits 1 / 2 / 3 / 4: .741 / .655 / .596 / .633; GPT-2 medium, 32 requests of mixed lengths, tokens a
    // second with 1 / 2 / 3 splits: 17-19 k / 21-23 k / 21 k).
    const int pairs = std::max(1, n_tokens * n_heads);
    const int by_blocks = (4 * sms + pairs / 2) / pairs;
    const int by_length = std::min((max_kv + 255) / 256, (8 * sms) / pairs);
    const int want = std::max(by_blocks, by_length);
    const int cap = std::max(1, max_kv / 64);
    const int n = std::max(1, std::min({want, cap, 32}));
    // The splits of a pair are one thread-block cluster.  Clusters of 6 and 7 blocks pack badly into
    // the GPU's groups of SMs: a whole decode step of 8 x 12 pairs took 0.439 / 0.441 ms with them
    // against 0.376 ms with 5 (0.383 with 4, 0.420 with 8).
    return (n == 6 || n == 7) ? 5 : n;
}

namespace {
constexpr int kClusterMaxSplits = 8;
// From this many (token, head) pairs on, a decode step's attention streams pages through shared
// memory with bulk copies (attention_decode_bulk.cu) instead of through registers.  Measured on
// GPT-2 small's shape: 64 x 12 pairs of 384 keys, cache read from HBM, 18.8 against 45.5 us a layer;
// but a whole decode step of 8 x 12 pairs (its cache fits in L2) took 414 against 400 us and one of
// 1 x 12 pairs 356 against 333 us, the register kernel starting sooner.
constexpr int kBulkMinPairs = 256;

bool decode_head_dim(DType dt, int d) {
    if (d == 16 || d == 32 || d == 64 || d == 128) return true;
    return d == 256 && dt == DType::BF16;
}
}  // namespace

void attention(const Launch& l, const AttentionStep& s, const Tensor& q, const KVView& c, Tensor& out, int n_heads,
               float scale, int window, Workspace& ws, const AttentionExtras* extras) {
    (void)ws;
    const float* sk = extras ? extras->sink : nullptr;
    const float* og = extras ? extras->out_gate : nullptr;
    const float cap = extras ? extras->softcap : 0.0f;
    const int chunk = extras ? extras->chunk : 0;
    if (cap < 0.0f || chunk < 0) throw UnsupportedShape("attention: softcap and chunk must not be negative");
    const float* db = extras ? extras->dist_bias : nullptr;
    const int n_dist = extras ? extras->n_dist : 0;
    if (db && n_dist < 1) throw UnsupportedShape("attention: a bias by distance needs at least one row");
    const bool ruled = cap > 0.0f || chunk > 0;           // only kernels with a form for these rules take such steps
    const int d = c.head_dim, hkv = c.n_kv_heads;
    if (d % 16 != 0 || d > kMaxHeadDim) throw UnsupportedShape("attention: head size " + std::to_string(d) + " must be a multiple of 16, at most " + std::to_string(kMaxHeadDim));
    if (hkv <= 0 || n_heads % hkv != 0)
        throw UnsupportedShape("attention: " + std::to_string(n_heads) + " heads do not divide into " + std::to_string(hkv) + " key/value heads");
    if (q.cols != (int64_t)n_heads * d || out.rows != q.rows || out.cols != q.cols || q.dtype != c.dtype || out.dtype != q.dtype)
        throw KernelError("attention: q and out must be [T, H*D] of the cache's dtype");
    const int T = (int)q.rows;
    if (left_out("attention")) return;
    const double attn_bytes = 2.0 * s.kv_tokens * hkv * d * q.elem_size() + 2 * tensor_bytes(&q);
    const double attn_flops = 4.0 * s.pairs * n_heads * d;
    const std::string shape = "(H=" + std::to_string(n_heads) + ",Hkv=" + std::to_string(hkv) + ",D=" + std::to_string(d) + ")";
    if (s.max_q_len > 1 && q.dtype == DType::BF16 && d <= 128) {
        static const bool use_tc = env_int("SANDYRT_PREFILL_TC", 1) != 0;     // 0 keeps every head size on the mma.sync kernel
        if (use_tc && d == 64 && !db) {                       // (the tcgen05 kernel has no form for a bias by distance)
            static auto fn = SANDY_KERNEL(attention_prefill_tc, sandy_prefill_attention_tc_cap);
            OpTimer timer(l, "attention, prompt (tcgen05)", attn_bytes, attn_flops);
            const int code = fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.q_start, s.kv_before,
                                out.data, (int)out.ld, s.n_seqs, s.max_q_len, n_heads, hkv, d, c.page_size, scale, window,
                                cap, chunk, c.num_pages, sk, og, l.kernel_status, l.stream);
            if (code != -1) { check(code, "prefill_attention_tc" + shape); return; }
        }
        static auto fn = SANDY_KERNEL(attention_prefill, sandy_prefill_attention_bias);
        OpTimer timer(l, "attention, prompt (mma.sync)", attn_bytes, attn_flops);
        check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.q_start, s.kv_before, out.data,
                 (int)out.ld, s.n_seqs, s.max_q_len, n_heads, hkv, d, c.page_size, scale, window, cap, chunk, c.num_pages, sk, og,
                 db, n_dist, l.kernel_status, l.stream),
              "prefill_attention" + shape);
        return;
    }
    // Many query heads on one key/value head (attention over a latent, few key/value heads): the heads as the rows
    // of the tensor-core instruction, keys fetched once per sixteen heads (attention_decode_shared.cu).  Blocks of
    // (token, group, sixteen heads) are few, so the keys are cut into enough splits for two blocks an SM, but no
    // split shorter than four groups of 16 keys (a warp each).
    // It is two launches with a floor of 9 us, so it takes the steps with enough (token, head, key) triples.  Alone, 12
    // heads of 128 on one key/value head, us, this kernel / the best of the kernels below: 1 token x 392 keys 9.1 / 5.2;
    // 8 x 392: 9.4 / 8.7; 8 tokens x 24 heads x 392: 11.3 / 16.6; 8 x 12 x 2,000: 13.2 / 36.2.
    // Steps with capped scores, chunks of positions or a bias by distance: this kernel is the decode kernel that has a form
    // for them, so it takes them all (with few keys it is one launch of one split); a chunk bounds the keys a query walks.
    if (s.max_q_len == 1 && q.dtype == DType::BF16 && d <= 128 && T <= 65535 &&
        (ruled || db || (n_heads / hkv >= kSharedKvMinHeads && (int64_t)T * n_heads * s.max_blocks * c.page_size >= kSharedKvMinTriples))) {
        const int max_kv = chunk > 0 ? std::min(chunk, s.max_blocks * c.page_size) : s.max_blocks * c.page_size;
        const int tiles = hkv * ((n_heads / hkv + 15) / 16), groups = (max_kv + 15) / 16;
        const int splits = std::max(1, std::min({(groups + 3) / 4, (2 * sm_count() + T * tiles - 1) / (T * tiles), 64}));
        static auto need = SANDY_KERNEL(attention_decode_shared, sandy_decode_attention_shared_scratch);
        static auto fn = SANDY_KERNEL(attention_decode_shared, sandy_decode_attention_shared_bias);
        const long long floats = need(T, n_heads, hkv, d, splits);
        float* scratch = floats ? (float*)ws.raw("decode_attention_partial_rows", (size_t)floats * sizeof(float)) : nullptr;
        OpTimer timer(l, "attention, decode (heads as rows)", attn_bytes, attn_flops);
        check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data, (int)out.ld,
                 T, n_heads, hkv, d, c.page_size, scale, window, cap, chunk, splits, c.num_pages, sk, og, db, n_dist, scratch,
                 l.kernel_status, l.stream),
              "decode_attention_shared" + shape);
        return;
    }
    if (!db && !ruled && s.max_q_len == 1 && decode_head_dim(q.dtype, d)) {
        const int max_kv = s.max_blocks * c.page_size;
        const int splits = std::min(decode_splits(T, n_heads, max_kv), kClusterMaxSplits);
        const size_t stage = 2 * (size_t)c.page_size * (size_t)d * q.elem_size();
        const bool fits = stage * 4 <= 160 * 1024;           // the ring holds at least four stages
        static const int bulk_mode = env_int("SANDYRT_DECODE_BULK", -1);      // 0 / 1 force one kernel, for comparisons
        const bool bulk = fits && (bulk_mode < 0 ? T * n_heads >= kBulkMinPairs : bulk_mode == 1);
        // bfloat16 heads of 64: the products on mma.sync (attention_decode_mma.cu).  Timed alone on caches from
        // HBM, 12 heads, 400 keys (us; register / bulk / mma.sync kernel): 1 token 4.5 / 5.2 / 3.4; 8 tokens 6.0 /
        // 7.5 / 5.1; 24 tokens 15.9 / 17.4 / 11.7; 48 tokens 25.9 / 23.2 / 16.0; 64 tokens 45 / 17.5 / 19.9; and
        // 8 tokens of 1,000 keys 12.9 / 12.5 / 7.8.  So it takes every launch but those with so many pairs that
        // a pair is one block (one split), where the bulk kernel's deeper ring of pages keeps its small lead.
        static const int mma_mode = env_int("SANDYRT_DECODE_MMA", 1);          // 0 keeps the two kernels below, for comparisons
        if (mma_mode != 0 && q.dtype == DType::BF16 && d == 64 && !(bulk && splits == 1)) {
            static auto max_keys_fn = SANDY_KERNEL(attention_decode_mma, sandy_decode_attention_mma_max_keys);
            if (max_kv <= max_keys_fn(splits, c.page_size)) {
                static auto fn = SANDY_KERNEL(attention_decode_mma, sandy_decode_attention_mma_ext);
                OpTimer timer(l, "attention, decode (mma.sync)", attn_bytes, attn_flops);
                check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                         (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, max_kv, sk, og, l.kernel_status,
                         l.stream),
                      "decode_attention_mma" + shape);
                return;
            }
        }
        if (bulk) {
            static auto fn = SANDY_KERNEL(attention_decode_bulk, sandy_decode_attention_bulk_ext);
            OpTimer timer(l, "attention, decode (bulk copies)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, code_of(q.dtype),
                     sk, og, l.kernel_status, l.stream),
                  "decode_attention_bulk" + shape);
        } else if (splits > 1) {
            static auto fn = SANDY_KERNEL(attention_decode, sandy_decode_attention_cluster_ext);
            OpTimer timer(l, "attention, decode (cluster)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, splits, c.num_pages, code_of(q.dtype),
                     sk, og, l.kernel_status, l.stream),
                  "decode_attention_cluster" + shape);
        } else {
            static auto fn = SANDY_KERNEL(attention_decode, sandy_decode_attention_ext);
            OpTimer timer(l, "attention, decode (one block)", attn_bytes, attn_flops);
            check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
                     (int)out.ld, nullptr, T, n_heads, hkv, d, c.page_size, scale, window, 1, c.num_pages, code_of(q.dtype),
                     sk, og, l.kernel_status, l.stream),
                  "decode_attention" + shape);
        }
        return;
    }
    static auto fn = SANDY_KERNEL(attention, sandy_paged_attention_bias);
    OpTimer timer(l, "attention, general", attn_bytes, attn_flops);
    check(fn(q.data, (int)q.ld, c.k, c.v, c.page_stride, s.block_table, s.max_blocks, s.token_seq, s.positions, out.data,
             (int)out.ld, T, n_heads, hkv, d, c.page_size, scale, window, cap, chunk, c.num_pages, code_of(q.dtype), sk, og, db,
             n_dist, l.kernel_status, l.stream),
          "paged_attention" + shape);
}

// ---- RMS norms, gates, casts ---------------------------------------------------------------------------
void rmsnorm(const Launch& l, const Tensor& x, const Tensor* gain, float eps, Tensor& out, const int* rows, int n_rows) {
    if (x.dtype != DType::F32 || (gain && (gain->dtype != DType::F32 || gain->numel() != x.cols)) || out.cols != x.cols ||
        out.rows < n_rows || (!rows && x.rows < n_rows))
        throw KernelError("rmsnorm: float32 x [rows, width], float32 gain [width], out [n_rows, width] expected");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(rmsnorm, sandy_rmsnorm);
    OpTimer timer(l, "rmsnorm", (double)n_rows * x.cols * (x.elem_size() + out.elem_size()), 0);
    check(fn((const float*)x.data, (int)x.ld, gain ? (const float*)gain->data : nullptr, out.data, (int)out.ld, rows, n_rows,
             (int)x.cols, eps, code_of(out.dtype), l.stream),
          "rmsnorm(width=" + std::to_string(x.cols) + ")");
}

void rmsnorm_shift(const Launch& l, const StepSeqs& s, const Tensor& x, const Tensor* gain, float eps, const Tensor& mix,
                   const StateView& state, Tensor& out, int max_q_len) {
    if (x.dtype != DType::F32 || (gain && (gain->dtype != DType::F32 || gain->numel() != x.cols)) || mix.dtype != DType::F32 ||
        mix.numel() != x.cols || out.rows != x.rows || out.cols != x.cols || state.dtype != DType::F32 || state.row_elems < x.cols ||
        x.rows != s.n_tokens)
        throw KernelError("rmsnorm_shift: float32 x [T, width], gain and mix [width], a float32 state of at least width floats expected");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(rmsnorm, sandy_rmsnorm_shift);
    static auto keep = SANDY_KERNEL(rmsnorm, sandy_rmsnorm_keep);
    const float* g = gain ? (const float*)gain->data : nullptr;
    {
        OpTimer timer(l, "rmsnorm + token shift", (double)x.rows * x.cols * (2 * x.elem_size() + out.elem_size()), 0);
        check(fn((const float*)x.data, (int)x.ld, g, (const float*)mix.data, (float*)state.data, (long long)state.row_elems,
                 s.token_seq, s.q_start, s.seq_slots, out.data, (int)out.ld, s.n_tokens, (int)x.cols, eps, code_of(out.dtype), l.stream),
              "rmsnorm_shift(width=" + std::to_string(x.cols) + ")");
    }
    if (max_q_len > 1) {
        OpTimer timer(l, "token shift: last rows kept", 2.0 * s.n_seqs * x.cols * sizeof(float), 0);
        check(keep((const float*)x.data, (int)x.ld, g, (float*)state.data, (long long)state.row_elems, s.q_start, s.seq_slots, s.n_seqs,
                   (int)x.cols, eps, l.stream),
              "rmsnorm_keep");
    }
}

void rmsnorm_add(const Launch& l, const Tensor& y, const Tensor* gain, float eps, float mult, Tensor& x) {
    if (x.dtype != DType::F32 || y.dtype != DType::F32 || x.rows != y.rows || x.cols != y.cols ||
        (gain && (gain->dtype != DType::F32 || gain->numel() != x.cols)))
        throw KernelError("rmsnorm_add: float32 x and y of one shape, float32 gain [width] expected");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(rmsnorm, sandy_rmsnorm_add);
    OpTimer timer(l, "rmsnorm + residual", 3.0 * tensor_bytes(&x), 0);
    check(fn((const float*)y.data, (int)y.ld, gain ? (const float*)gain->data : nullptr, (float*)x.data, (int)x.ld, (int)x.rows,
             (int)x.cols, eps, mult, l.stream),
          "rmsnorm_add(width=" + std::to_string(x.cols) + ")");
}

void head_norm_gate(const Launch& l, const Tensor& o, const Tensor* gain, const Tensor* gate, GateAct act, float scale,
                    float eps, int n_heads, Tensor& out) {
    if (n_heads <= 0 || o.cols % n_heads) throw KernelError("head_norm_gate: the columns do not divide into the heads");
    const int dim = (int)(o.cols / n_heads);
    if (o.dtype != DType::F32 || out.rows != o.rows || out.cols != o.cols ||
        (gain && (gain->dtype != DType::F32 || (gain->numel() != dim && gain->numel() != o.cols))) ||
        (gate && (gate->rows != o.rows || gate->cols != o.cols)))
        throw KernelError("head_norm_gate: float32 o [T, H * dim], gain [dim] or [H * dim], gate and out [T, H * dim] expected");
    static auto fn = SANDY_KERNEL(rmsnorm, sandy_head_norm_gate);
    OpTimer timer(l, "head norm + gate", tensor_bytes(&o) + tensor_bytes(gate) + tensor_bytes(&out), 0);
    check(fn((const float*)o.data, (int)o.ld, gain ? (const float*)gain->data : nullptr,
             gain && gain->numel() == o.cols && n_heads > 1 ? dim : 0, gate ? gate->data : nullptr, gate ? (int)gate->ld : 0,
             gate ? code_of(gate->dtype) : code_of(out.dtype), out.data, (int)out.ld, code_of(out.dtype), (int)o.rows, n_heads,
             dim, eps, (int)act, scale, l.stream),
          "head_norm_gate(H=" + std::to_string(n_heads) + ",dim=" + std::to_string(dim) + ")");
}

void glu(const Launch& l, const Tensor& a, const Tensor& b, GluAct act, Tensor& out) {
    if (a.dtype != b.dtype || a.dtype != out.dtype || a.rows != b.rows || a.cols != b.cols || a.ld != b.ld || out.rows != a.rows ||
        out.cols != a.cols)
        throw KernelError("glu: a, b and out must agree in shape and type");
    static auto fn = SANDY_KERNEL(elementwise, sandy_glu);
    OpTimer timer(l, "gated activation", 3.0 * tensor_bytes(&out), 0);
    check(fn(a.data, b.data, (int)a.ld, out.data, (int)out.ld, (int)a.rows, (int)a.cols, (int)act, code_of(a.dtype), l.stream), "glu");
}

void glu_clamped(const Launch& l, const Tensor& a, const Tensor& b, float limit, float alpha, Tensor& out) {
    if (a.dtype != b.dtype || a.dtype != out.dtype || a.rows != b.rows || a.cols != b.cols || a.ld != b.ld || out.rows != a.rows ||
        out.cols != a.cols)
        throw KernelError("glu_clamped: a, b and out must agree in shape and type");
    static auto fn = SANDY_KERNEL(elementwise, sandy_glu_clamped);
    OpTimer timer(l, "gated activation", 3.0 * tensor_bytes(&out), 0);
    check(fn(a.data, b.data, (int)a.ld, out.data, (int)out.ld, (int)a.rows, (int)a.cols, limit, alpha, code_of(a.dtype), l.stream),
          "glu_clamped");
}

void stream_add(const Launch& l, Tensor& x, const Tensor* x0, const Tensor* row) {
    if (x.dtype != DType::F32 || (x0 && (x0->dtype != DType::F32 || x0->rows != x.rows || x0->cols != x.cols)) ||
        (row && (row->dtype != DType::F32 || row->numel() != x.cols)))
        throw KernelError("stream_add: float32 x and x0 of one shape, a float32 row [width] expected");
    static auto fn = SANDY_KERNEL(elementwise, sandy_stream_add);
    OpTimer timer(l, "stream + embedding + row", (x0 ? 3.0 : 2.0) * tensor_bytes(&x), 0);
    check(fn((float*)x.data, (int)x.ld, x0 ? (const float*)x0->data : nullptr, x0 ? (int)x0->ld : 0,
             row ? (const float*)row->data : nullptr, (int)x.rows, (int)x.cols, l.stream),
          "stream_add");
}

void softcap(const Launch& l, Tensor& x, float cap) {
    if (x.dtype != DType::F32 || !x.contiguous()) throw KernelError("softcap: a dense float32 tensor expected");
    static auto fn = SANDY_KERNEL(elementwise, sandy_softcap_f32);
    OpTimer timer(l, "softcap", 2.0 * tensor_bytes(&x), 0);
    check(fn((float*)x.data, (long long)x.numel(), cap, l.stream), "softcap");
}

void cast_cols(const Launch& l, const Tensor& x, Tensor& out) {
    if (x.dtype != DType::F32 || out.rows != x.rows || out.cols != x.cols) throw KernelError("cast_cols: float32 x and out of one shape expected");
    static auto fn = SANDY_KERNEL(elementwise, sandy_cast_cols);
    OpTimer timer(l, "cast", tensor_bytes(&x) + tensor_bytes(&out), 0);
    check(fn((const float*)x.data, (int)x.ld, out.data, (int)out.ld, (int)x.rows, (int)x.cols, code_of(out.dtype), l.stream), "cast_cols");
}

void scale_add(const Launch& l, const Tensor& y, const Tensor& gain, const Tensor* y2, const Tensor* gain2, Tensor& x) {
    if (x.dtype != DType::F32 || y.dtype != DType::F32 || gain.dtype != DType::F32 || y.rows != x.rows || y.cols != x.cols ||
        gain.numel() != x.cols || (y2 && (!gain2 || y2->dtype != DType::F32 || gain2->dtype != DType::F32 || y2->rows != x.rows ||
                                          y2->cols != x.cols || gain2->numel() != x.cols)))
        throw KernelError("scale_add: float32 x and y of one shape, float32 gain [width] expected");
    static auto fn = SANDY_KERNEL(elementwise, sandy_scale_add);
    OpTimer timer(l, "layer scale + residual", (y2 ? 4.0 : 3.0) * tensor_bytes(&x), 0);
    check(fn((const float*)y.data, (int)y.ld, (const float*)gain.data, y2 ? (const float*)y2->data : nullptr, y2 ? (int)y2->ld : 0,
             y2 ? (const float*)gain2->data : nullptr, (float*)x.data, (int)x.ld, (int)x.rows, (int)x.cols, l.stream),
          "scale_add");
}

void scale(const Launch& l, Tensor& x, float s) {
    if (x.dtype != DType::F32 || !x.contiguous()) throw KernelError("scale: a dense float32 tensor expected");
    static auto fn = SANDY_KERNEL(elementwise, sandy_scale_f32);
    OpTimer timer(l, "scale", 2.0 * tensor_bytes(&x), 0);
    check(fn((float*)x.data, (long long)x.numel(), s, l.stream), "scale");
}

void latent_prepare(const Launch& l, const LatentPrepare& p, const Tensor& down, const Tensor* q, const KVView& c,
                    const int* block_table, int max_blocks, const int* token_seq, const int* positions, Tensor* q_latent,
                    Tensor& q_abs) {
    const int64_t T = down.rows;
    if (down.dtype != DType::F32 || down.cols < p.q_rank + p.kv_rank + p.rot_dim || c.n_kv_heads != 1 || c.k != c.v ||
        c.head_dim < p.kv_rank + p.rot_dim || q_abs.dtype != c.dtype || q_abs.rows != T ||
        q_abs.cols != (int64_t)p.n_heads * c.head_dim ||
        (p.rot_dim > 0 && (!q || q->dtype != c.dtype || q->rows != T || q->cols != (int64_t)p.n_heads * (p.qk_dim + p.rot_dim))) ||
        (p.q_rank > 0 && (!q_latent || q_latent->dtype != c.dtype || q_latent->rows != T || q_latent->cols != p.q_rank)))
        throw KernelError("latent_prepare: the projections, the queries and the one-plane cache disagree");
    static auto fn = SANDY_KERNEL(latent_prepare, sandy_latent_prepare);
    OpTimer timer(l, "latent norm + rotary + cache write", tensor_bytes(&down) + (double)T * c.head_dim * (p.n_heads + 1) * q_abs.elem_size(), 0);
    check(fn((const float*)down.data, (int)down.ld, (int)T, p.q_rank, p.kv_rank, p.rot_dim, p.q_gain, p.kv_gain, p.eps, p.freq,
             p.rot_dims, positions, token_seq, block_table, max_blocks, c.k, c.page_stride, c.page_size, c.num_pages, c.head_dim,
             p.write_cache ? 1 : 0, q_latent ? q_latent->data : nullptr, q_latent ? (int)q_latent->ld : 0, q ? q->data : nullptr,
             q ? (int)q->ld : 0, p.n_heads, p.qk_dim, q_abs.data, (int)q_abs.ld, code_of(c.dtype), l.kernel_status, l.stream),
          "latent_prepare");
}

void head_product(const Launch& l, const Tensor& a, int a_gcols, const Tensor& w, int n_groups, Tensor& out, int o_gcols) {
    if (n_groups <= 0 || w.rows % n_groups) throw KernelError("head_product: the weight's rows do not divide into the heads");
    const int64_t N = w.rows / n_groups, K = w.cols;
    if (a.dtype != w.dtype || a.rows != out.rows || a.cols < (int64_t)(n_groups - 1) * a_gcols + K ||
        out.cols < (int64_t)(n_groups - 1) * o_gcols + N || (out.dtype != a.dtype && out.dtype != DType::F32))
        throw KernelError("head_product: a " + dims(a) + ", w " + dims(w) + " and out " + dims(out) + " disagree");
    if (left_out("product", N, K)) return;
    static auto fn = SANDY_KERNEL(grouped_gemm, sandy_head_product);
    OpTimer timer(l, "product per head", tensor_bytes(&w) + (double)a.rows * n_groups * (K * a.elem_size() + N * out.elem_size()),
                  2.0 * a.rows * n_groups * N * K);
    check(fn(a.data, (int)a.ld, a_gcols, w.data, (long long)N * w.ld, (int)w.ld, out.data, (int)out.ld, o_gcols, (int)a.rows, n_groups,
             (int)N, (int)K, code_of(a.dtype), code_of(out.dtype), l.stream),
          "head_product(G=" + std::to_string(n_groups) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
}

void moe_route(const Launch& l, const Tensor& logits, const Tensor* bias, const Routing& r) {
    if (logits.dtype != DType::F32 || logits.rows != r.n_tokens || logits.cols != r.n_experts ||
        (bias && (bias->dtype != DType::F32 || bias->numel() != r.n_experts)))
        throw KernelError("moe_route: float32 logits [tokens, experts] and a float32 bias [experts] expected");
    static auto route = SANDY_KERNEL(moe, sandy_moe_route);
    static auto group = SANDY_KERNEL(moe, sandy_moe_group);
    {
        OpTimer timer(l, "expert routing", tensor_bytes(&logits), 0);
        check(route((const float*)logits.data, (int)logits.ld, bias ? (const float*)bias->data : nullptr, r.n_tokens, r.n_experts, r.top,
                    r.expert_of, r.weight_of, l.stream),
              "moe_route(E=" + std::to_string(r.n_experts) + ",top=" + std::to_string(r.top) + ")");
    }
    OpTimer timer(l, "expert grouping", 12.0 * r.n_tokens * r.top, 0);
    check(group(r.expert_of, r.n_tokens * r.top, r.n_experts, r.group_start, r.entry_of_slot, r.slot_of_entry, l.stream), "moe_group");
}

void moe_route_scored(const Launch& l, const Tensor& logits, const Tensor* correction, const ScoredRoute& rule, const Routing& r) {
    if (logits.dtype != DType::F32 || logits.rows != r.n_tokens || logits.cols != r.n_experts ||
        (correction && (correction->dtype != DType::F32 || correction->numel() != r.n_experts)))
        throw KernelError("moe_route_scored: float32 logits [tokens, experts] and a float32 correction [experts] expected");
    static auto route = SANDY_KERNEL(moe, sandy_moe_route_scored);
    static auto group = SANDY_KERNEL(moe, sandy_moe_group);
    {
        OpTimer timer(l, "expert routing", tensor_bytes(&logits), 0);
        check(route((const float*)logits.data, (int)logits.ld, correction ? (const float*)correction->data : nullptr, r.n_tokens,
                    r.n_experts, r.top, rule.n_groups, rule.keep_groups, rule.group_rank, rule.weight_scale, rule.norm_eps, r.expert_of,
                    r.weight_of, l.stream),
              "moe_route_scored(E=" + std::to_string(r.n_experts) + ",top=" + std::to_string(r.top) + ",groups=" +
                  std::to_string(rule.n_groups) + ")");
    }
    OpTimer timer(l, "expert grouping", 12.0 * r.n_tokens * r.top, 0);
    check(group(r.expert_of, r.n_tokens * r.top, r.n_experts, r.group_start, r.entry_of_slot, r.slot_of_entry, l.stream), "moe_group");
}

void moe_route_softmax(const Launch& l, const Tensor& logits, const Tensor* correction, const SoftmaxRoute& rule, const Routing& r) {
    if (logits.dtype != DType::F32 || logits.rows != r.n_tokens || logits.cols != r.n_experts ||
        (correction && (correction->dtype != DType::F32 || correction->numel() != r.n_experts)))
        throw KernelError("moe_route_softmax: float32 logits [tokens, experts] and a float32 correction [experts] expected");
    static auto route = SANDY_KERNEL(moe, sandy_moe_route_softmax);
    static auto group = SANDY_KERNEL(moe, sandy_moe_group);
    {
        OpTimer timer(l, "expert routing", tensor_bytes(&logits), 0);
        check(route((const float*)logits.data, (int)logits.ld, correction ? (const float*)correction->data : nullptr, r.n_tokens,
                    r.n_experts, r.top, rule.weight_scale, rule.norm_eps, rule.renormalize ? 1 : 0, r.expert_of, r.weight_of, l.stream),
              "moe_route_softmax(E=" + std::to_string(r.n_experts) + ",top=" + std::to_string(r.top) + ")");
    }
    OpTimer timer(l, "expert grouping", 12.0 * r.n_tokens * r.top, 0);
    check(group(r.expert_of, r.n_tokens * r.top, r.n_experts, r.group_start, r.entry_of_slot, r.slot_of_entry, l.stream), "moe_group");
}

void expert_product(const Launch& l, const Routing& r, const Tensor& a, bool gather, const Tensor& w, ExpertAct act, Tensor& out,
                    Tensor* sorted) {
    if (r.n_experts <= 0 || w.rows % r.n_experts) throw KernelError("expert_product: the weight's rows do not divide into the experts");
    const int64_t N = w.rows / r.n_experts, K = w.cols, slots = (int64_t)r.n_tokens * r.top;
    if (a.dtype != w.dtype || a.cols != K || a.rows != (gather ? r.n_tokens : slots) || out.rows != slots || out.cols != N ||
        (out.dtype != a.dtype && out.dtype != DType::F32))
        throw KernelError("expert_product: a " + dims(a) + ", w " + dims(w) + " and out " + dims(out) + " disagree");
    if (left_out("product", N, K)) return;
    // bytes: every expert's matrix at most once, and no more matrices than slots
    const double matrices = std::min<double>(r.n_experts, (double)slots);
    static const int tc_mode = env_int("SANDYRT_EXPERT_TC", -1);      // 0 / 1 force one kernel, for comparisons
    if (tc_mode != 0 && a.dtype == DType::BF16 && K % 8 == 0 && w.ld % 8 == 0 && !((uintptr_t)w.data & 15) && (!gather || sorted)) {
        const Tensor* rows = &a;
        if (gather) {
            if (sorted->dtype != a.dtype || sorted->rows != slots || sorted->cols != K) throw KernelError("expert_product: the scratch for sorted rows must be [slots, K] of a's type");
            static auto gather_fn = SANDY_KERNEL(moe, sandy_moe_gather);
            OpTimer timer(l, "expert rows, sorted", 2.0 * tensor_bytes(sorted), 0);
            check(gather_fn(a.data, (long long)a.ld * (long long)a.elem_size(), r.entry_of_slot, r.top, sorted->data,
                            (long long)sorted->ld * (long long)sorted->elem_size(), (int)slots, (int)(K * a.elem_size()), l.stream),
                  "moe_gather");
            rows = sorted;
        }
        if (rows->ld % 8 == 0 && !((uintptr_t)rows->data & 15)) {
            static auto tc = SANDY_KERNEL(grouped_gemm_tc, sandy_expert_product_tc);
            OpTimer timer(l, "product per expert (tcgen05)", matrices * N * K * w.elem_size() + (double)slots * (K * a.elem_size() + N * out.elem_size()),
                          2.0 * slots * N * K);
            check(tc(rows->data, (int)rows->ld, w.data, (int)w.ld, out.data, (int)out.ld, (int)slots, r.n_experts, (int)N, (int)K, r.group_start,
                     (int)act, code_of(out.dtype), l.kernel_status, l.stream),
                  "expert_product_tc(E=" + std::to_string(r.n_experts) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
            return;
        }
    }
    static auto fn = SANDY_KERNEL(grouped_gemm, sandy_expert_product);
    OpTimer timer(l, "product per expert", matrices * N * K * w.elem_size() + (double)slots * (K * a.elem_size() + N * out.elem_size()),
                  2.0 * slots * N * K);
    check(fn(a.data, (int)a.ld, w.data, (long long)N * w.ld, (int)w.ld, out.data, (int)out.ld, (int)slots, r.n_experts, (int)N, (int)K,
             r.group_start, gather ? r.entry_of_slot : nullptr, gather ? r.top : 1, (int)act, code_of(a.dtype), code_of(out.dtype), l.stream),
          "expert_product(E=" + std::to_string(r.n_experts) + ",N=" + std::to_string(N) + ",K=" + std::to_string(K) + ")");
}

void moe_combine(const Launch& l, const Routing& r, const Tensor& rows, Tensor& y, bool add) {
    if (rows.dtype != DType::F32 || y.dtype != DType::F32 || rows.rows != (int64_t)r.n_tokens * r.top || y.rows != r.n_tokens ||
        rows.cols != y.cols)
        throw KernelError("moe_combine: float32 rows [tokens * top, width] and y [tokens, width] expected");
    static auto fn = SANDY_KERNEL(moe, sandy_moe_combine);
    OpTimer timer(l, "expert combine", tensor_bytes(&rows) + (add ? 2.0 : 1.0) * tensor_bytes(&y), 0);
    check(fn((const float*)rows.data, (int)rows.ld, r.weight_of, r.slot_of_entry, r.n_tokens, r.top, (float*)y.data, (int)y.ld,
             (int)y.cols, add ? 1 : 0, l.stream),
          "moe_combine");
}

void moe_combine_identity(const Launch& l, const Routing& r, int n_real, const Tensor& h, const Tensor& rows, Tensor& y, bool add) {
    if (rows.dtype != DType::F32 || y.dtype != DType::F32 || rows.rows != (int64_t)r.n_tokens * r.top || y.rows != r.n_tokens ||
        rows.cols != y.cols || h.rows != y.rows || h.cols != y.cols || (h.dtype != DType::F32 && h.dtype != DType::BF16))
        throw KernelError("moe_combine_identity: float32 rows [tokens * top, width], y and h [tokens, width] expected");
    static auto fn = SANDY_KERNEL(moe, sandy_moe_combine_identity);
    OpTimer timer(l, "expert combine", tensor_bytes(&rows) + (add ? 2.0 : 1.0) * tensor_bytes(&y) + tensor_bytes(&h), 0);
    check(fn((const float*)rows.data, (int)rows.ld, r.weight_of, r.slot_of_entry, r.expert_of, n_real, h.data, (int)h.ld,
             code_of(h.dtype), r.n_tokens, r.top, (float*)y.data, (int)y.ld, (int)y.cols, add ? 1 : 0, l.stream),
          "moe_combine_identity");
}

void attention_prepare(const Launch& l, const AttentionPrepare& p, const Tensor& proj, const KVView& c, const int* block_table,
                       int max_blocks, const int* token_seq, const int* positions, Tensor& q_out) {
    if (proj.dtype != c.dtype || q_out.dtype != proj.dtype || q_out.rows != proj.rows || q_out.cols != (int64_t)p.n_heads * c.head_dim ||
        c.n_kv_heads != p.n_kv_heads || c.head_dim < p.qk_dim || c.head_dim < p.v_dim)
        throw KernelError("attention_prepare: the projection, the queries and the cache disagree");
    static auto fn = SANDY_KERNEL(attention_prepare, sandy_attention_prepare_pos);
    OpTimer timer(l, "q/k norm + rotary + cache write", 2.0 * tensor_bytes(&proj), 0);
    check(fn(proj.data, (int)proj.ld, p.q_off, p.k_off, p.v_off, (int)proj.rows, p.n_heads, p.n_kv_heads, p.qk_dim, p.v_dim,
             c.head_dim, p.q_gain, p.k_gain, p.eps, p.freq, p.rot_dims, positions, token_seq, block_table, max_blocks, c.k, c.v,
             c.page_stride, c.page_size, c.num_pages, p.write_cache ? 1 : 0, q_out.data, (int)q_out.ld, p.gate_in, p.ld_gate,
             p.gate_out, p.gate_scale, p.q_head_scale, p.v_unit_eps, p.per_head_norm ? 1 : 0, p.q_pos_coef, p.q_pos_every,
             code_of(proj.dtype), l.kernel_status, l.stream),
          "attention_prepare");
}

// ---- recurrent mixers ------------------------------------------------------------------------------------
int64_t mlstm_state_floats(int n_heads, int qk_dim, int v_dim) {
    const int64_t Z = (v_dim + kMatrixStateCols - 1) / kMatrixStateCols;
    return (int64_t)n_heads * v_dim * qk_dim + (int64_t)n_heads * Z * qk_dim + (int64_t)n_heads * Z;
}

void delta_prepare(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& proj, const Tensor& taps,
                   const Tensor& gates, const float* a_log, const float* dt_bias, const StateView& state, int64_t tail_off,
                   float q_scale, Tensor& qkv, Tensor& bg) {
    const int64_t channels = 2 * (int64_t)d.n_qk_heads * d.qk_dim + (int64_t)d.n_heads * d.v_dim;
    if (proj.cols < channels || taps.dtype != DType::F32 || taps.numel() != channels * d.n_taps || gates.dtype != DType::F32 ||
        gates.cols < 2 * d.n_heads || qkv.dtype != DType::F32 || qkv.cols != channels || bg.dtype != DType::F32 ||
        bg.cols != 2 * d.n_heads || !bg.contiguous() || state.dtype != DType::F32)
        throw KernelError("delta_prepare: shapes disagree");
    static auto fn = SANDY_KERNEL(matrix_state, sandy_delta_prepare);
    OpTimer timer(l, "delta rule: conv + norms + gates", tensor_bytes(&proj) + tensor_bytes(&qkv), 0);
    check(fn(proj.data, (int)proj.ld, code_of(proj.dtype), (const float*)taps.data, d.n_taps, (const float*)gates.data, (int)gates.ld,
             a_log, dt_bias, (const float*)state.data, state.row_elems, tail_off, s.token_seq, s.q_start, s.seq_slots,
             (float*)qkv.data, (int)qkv.ld, (float*)bg.data, s.n_tokens, d.n_heads, d.n_qk_heads, d.qk_dim, d.v_dim, q_scale, l.stream),
          "delta_prepare");
}

void conv_tail(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& proj, const StateView& state, int64_t tail_off) {
    const int64_t channels = 2 * (int64_t)d.n_qk_heads * d.qk_dim + (int64_t)d.n_heads * d.v_dim;
    static auto fn = SANDY_KERNEL(matrix_state, sandy_conv_tail);
    OpTimer timer(l, "delta rule: conv tail", 0, 0);
    check(fn(proj.data, (int)proj.ld, code_of(proj.dtype), (int)channels, d.n_taps, (float*)state.data, state.row_elems, tail_off,
             s.q_start, s.seq_slots, s.n_seqs, l.stream),
          "conv_tail");
}

void conv_tail(const Launch& l, const StepSeqs& s, const Tensor& rows, int n_taps, const StateView& state, int64_t tail_off) {
    if (state.dtype != DType::F32 || n_taps < 1 || tail_off < 0 || tail_off + (int64_t)(n_taps - 1) * rows.cols > state.row_elems)
        throw KernelError("conv_tail: the tail does not fit the float32 state");
    if (n_taps == 1) return;
    static auto fn = SANDY_KERNEL(matrix_state, sandy_conv_tail);
    OpTimer timer(l, "conv tail", 0, 0);
    check(fn(rows.data, (int)rows.ld, code_of(rows.dtype), (int)rows.cols, n_taps, (float*)state.data, state.row_elems, tail_off,
             s.q_start, s.seq_slots, s.n_seqs, l.stream),
          "conv_tail");
}

// ---- selective state-space mixer -----------------------------------------------------------------------------
int64_t ssm_state_floats(const SsmShape& m) { return (int64_t)m.n_heads * m.v_dim * m.state; }

void ssm_prepare(const Launch& l, const StepSeqs& s, const SsmShape& m, const Tensor& proj, const Tensor& taps, const Tensor* conv_bias,
                 const Tensor& dt_raw, const float* dt_bias, const float* a_log, const StateView& state, int64_t tail_off,
                 Tensor& xbc, Tensor& dta, int max_q_len) {
    const int64_t channels = (int64_t)m.n_heads * m.v_dim + 2 * (int64_t)m.n_groups * m.state;
    if (proj.cols != channels || proj.rows != s.n_tokens || taps.dtype != DType::F32 || taps.numel() != channels * m.n_taps ||
        (conv_bias && (conv_bias->dtype != DType::F32 || conv_bias->numel() != channels)) || dt_raw.dtype != DType::F32 ||
        dt_raw.cols != m.n_heads || dt_raw.rows != proj.rows || xbc.dtype != DType::F32 || xbc.cols != channels ||
        xbc.rows != proj.rows || dta.dtype != DType::F32 || dta.cols != 2 * m.n_heads || !dta.contiguous() ||
        state.dtype != DType::F32 || tail_off + (int64_t)(m.n_taps - 1) * channels > state.row_elems)
        throw KernelError("ssm_prepare: shapes disagree");
    static auto fn = SANDY_KERNEL(ssm_state, sandy_ssm_prepare);
    {
        OpTimer timer(l, "state space: conv + gates", tensor_bytes(&proj) + tensor_bytes(&xbc), 0);
        check(fn(proj.data, (int)proj.ld, code_of(proj.dtype), (int)channels, (const float*)taps.data, m.n_taps,
                 conv_bias ? (const float*)conv_bias->data : nullptr, (const float*)dt_raw.data, (int)dt_raw.ld, dt_bias, a_log,
                 m.n_heads, (float*)state.data, state.row_elems, tail_off, s.token_seq, s.q_start, s.seq_slots, (float*)xbc.data,
                 (int)xbc.ld, (float*)dta.data, s.n_tokens, max_q_len <= 1 ? 1 : 0, l.stream),
              "ssm_prepare");
    }
    if (max_q_len > 1) conv_tail(l, s, proj, m.n_taps, state, tail_off);
}

void ssm_scan(const Launch& l, const StepSeqs& s, const SsmShape& m, const Tensor& xbc, const Tensor& dta, const float* d_skip,
              const StateView& state, Tensor& out) {
    if (out.dtype != DType::F32 || out.cols != (int64_t)m.n_heads * m.v_dim || xbc.dtype != DType::F32 || dta.dtype != DType::F32 ||
        !dta.contiguous() || state.dtype != DType::F32 || ssm_state_floats(m) > state.row_elems)
        throw KernelError("ssm_scan: float32 xbc, dta, out [T, H * P] and a float32 state of H * P * N floats expected");
    static auto fn = SANDY_KERNEL(ssm_state, sandy_ssm_scan);
    const double st = 2.0 * s.n_seqs * (double)ssm_state_floats(m) * 4.0;
    OpTimer timer(l, "state space: recurrence", st + tensor_bytes(&xbc) + tensor_bytes(&out), 6.0 * s.n_tokens * (double)ssm_state_floats(m));
    check(fn((const float*)xbc.data, (int)xbc.ld, (const float*)dta.data, d_skip, (float*)state.data, state.row_elems, s.q_start,
             s.seq_slots, (float*)out.data, (int)out.ld, s.n_seqs, m.n_heads, m.n_groups, m.state, m.v_dim, l.stream),
          "ssm_scan(H=" + std::to_string(m.n_heads) + ",N=" + std::to_string(m.state) + ",P=" + std::to_string(m.v_dim) + ")");
}

void gated_group_norm(const Launch& l, const Tensor& y, const Tensor& z, const Tensor* gain, float eps, int groups, Tensor& out) {
    if (y.dtype != DType::F32 || z.rows != y.rows || z.cols != y.cols || out.rows != y.rows || out.cols != y.cols || out.dtype != z.dtype ||
        groups < 1 || y.cols % groups || (gain && (gain->dtype != DType::F32 || gain->numel() != y.cols)))
        throw KernelError("gated_group_norm: float32 y, z and out [T, cols] of one type, float32 gain [cols] expected");
    static auto fn = SANDY_KERNEL(ssm_state, sandy_gated_group_norm);
    OpTimer timer(l, "gate + group norm", tensor_bytes(&y) + tensor_bytes(&z) + tensor_bytes(&out), 0);
    check(fn((const float*)y.data, (int)y.ld, z.data, (int)z.ld, gain ? (const float*)gain->data : nullptr, eps, groups, out.data,
             (int)out.ld, (int)y.rows, (int)y.cols, code_of(out.dtype), l.stream),
          "gated_group_norm");
}

// ---- a residual stream in several copies ----------------------------------------------------------------------
int streams_max() {
    static auto fn = SANDY_KERNEL(streams, sandy_streams_max);
    return fn();
}

void streams_step(const Launch& l, Tensor& X, int n_streams, const StreamsStep& p) {
    if (X.dtype != DType::F32 || n_streams < 1 || X.cols % n_streams) throw KernelError("streams_step: float32 streams [T, S * width] expected");
    const int64_t W = X.cols / n_streams;
    auto f32 = [](const Tensor* t, int64_t n) { return t && t->dtype == DType::F32 && t->numel() == n; };
    if (p.y && (p.y->dtype != DType::F32 || p.y->rows != X.rows || p.y->cols != W || !p.gate || p.gate->dtype != DType::F32 ||
                p.gate->rows != X.rows || p.gate->cols != W || !f32(p.gate_bias, W) || !f32(p.mix, (int64_t)n_streams * n_streams) ||
                !f32(p.out_w, n_streams)))
        throw KernelError("streams_step: the write needs float32 y and gate [T, width], gate_bias [width], mix [S, S] and out [S]");
    if (p.in_w && (!f32(p.in_w, n_streams) || !f32(p.gain, W) || !p.h || p.h->rows != X.rows || p.h->cols != W))
        throw KernelError("streams_step: the read needs float32 in [S] and gain [width] and h [T, width]");
    if (p.sum_out && (p.sum_out->dtype != DType::F32 || p.sum_out->rows != X.rows || p.sum_out->cols != W))
        throw KernelError("streams_step: the sum is float32 [T, width]");
    if (p.taps && (!p.in_w || !p.conv_out || p.conv_out->rows != X.rows || p.conv_out->cols != W || p.conv_out->dtype != p.h->dtype ||
                   !f32(p.taps, W * p.n_taps) || !p.seqs || p.seqs->n_tokens != X.rows ||
                   (p.n_taps > 1 && (!p.state || p.state->dtype != DType::F32 || p.tail_off + (int64_t)(p.n_taps - 1) * W > p.state->row_elems))))
        throw KernelError("streams_step: the convolution needs the read, float32 taps [width, n_taps], its output and a float32 state");
    if (left_out("layernorm")) return;
    static auto fn = SANDY_KERNEL(streams, sandy_streams_step_conv);
    OpTimer timer(l, "streams: write + norm", (p.y ? 2.0 : 1.0) * tensor_bytes(&X) + 2 * tensor_bytes(p.y) + tensor_bytes(p.h) + tensor_bytes(p.sum_out), 0);
    check(fn((float*)X.data, (int)X.ld, (int)X.rows, n_streams, (int)W, p.y ? (const float*)p.y->data : nullptr, p.y ? (int)p.y->ld : 0,
             p.y ? (const float*)p.gate->data : nullptr, p.y ? (int)p.gate->ld : 0, p.y ? (const float*)p.gate_bias->data : nullptr,
             p.y ? (const float*)p.mix->data : nullptr, p.y ? (const float*)p.out_w->data : nullptr,
             p.in_w ? (const float*)p.in_w->data : nullptr, p.in_w ? (const float*)p.gain->data : nullptr, p.eps,
             p.in_w ? p.h->data : nullptr, p.in_w ? (int)p.h->ld : 0, p.in_w ? code_of(p.h->dtype) : 0,
             p.sum_out ? (float*)p.sum_out->data : nullptr, p.sum_out ? (int)p.sum_out->ld : 0,
             p.taps ? (const float*)p.taps->data : nullptr, p.taps ? p.n_taps : 0, p.taps && p.state ? (float*)p.state->data : nullptr,
             p.taps && p.state ? p.state->row_elems : 0, p.tail_off, p.taps ? p.seqs->token_seq : nullptr,
             p.taps ? p.seqs->seq_slots : nullptr, p.taps ? p.conv_out->data : nullptr, p.taps ? (int)p.conv_out->ld : 0, l.stream),
          "streams_step(S=" + std::to_string(n_streams) + ",width=" + std::to_string(W) + ")");
}

void streams_spread(const Launch& l, const Tensor& x, Tensor& X, int n_streams) {
    if (x.dtype != DType::F32 || X.dtype != DType::F32 || X.rows != x.rows || X.cols != x.cols * n_streams)
        throw KernelError("streams_spread: float32 x [T, width] and X [T, S * width] expected");
    static auto fn = SANDY_KERNEL(streams, sandy_streams_spread);
    OpTimer timer(l, "streams: spread", tensor_bytes(&x) + tensor_bytes(&X), 0);
    check(fn((const float*)x.data, (int)x.ld, (float*)X.data, (int)X.ld, (int)x.rows, n_streams, (int)x.cols, l.stream), "streams_spread");
}

void canon_conv(const Launch& l, const StepSeqs& s, const Tensor& h, const Tensor& taps, int n_taps, const StateView& state,
                int64_t tail_off, Tensor& c) {
    if (h.dtype != c.dtype || h.rows != c.rows || h.cols != c.cols || h.rows != s.n_tokens || taps.dtype != DType::F32 ||
        taps.numel() != h.cols * n_taps || (n_taps > 1 && (state.dtype != DType::F32 || tail_off + (int64_t)(n_taps - 1) * h.cols > state.row_elems)))
        throw KernelError("canon_conv: h and c [T, width] of one type, float32 taps [width, n_taps] and a float32 state expected");
    static auto fn = SANDY_KERNEL(streams, sandy_canon_conv);
    OpTimer timer(l, "input conv", tensor_bytes(&h) + tensor_bytes(&c), 0);
    check(fn(h.data, (int)h.ld, (const float*)taps.data, n_taps, (const float*)state.data, state.row_elems, tail_off, s.token_seq,
             s.q_start, s.seq_slots, c.data, (int)c.ld, (int)h.rows, (int)h.cols, code_of(h.dtype), l.stream),
          "canon_conv");
}

void embed_bigram(const Launch& l, const StepSeqs& s, const int* ids, const int* positions, const Tensor& wte, const Tensor& bigram,
                  const Tensor* wpe, const BigramEmbed& b, const StateView& state, Tensor& x, int max_q_len) {
    if (x.dtype != DType::F32 || x.cols != wte.cols || bigram.dtype != wte.dtype || bigram.cols != wte.cols || bigram.rows != b.buckets + 1 ||
        (wpe && (wpe->dtype != wte.dtype || wpe->cols != wte.cols)) || state.dtype != DType::I32 || state.row_elems < 1 ||
        !wte.contiguous() || !bigram.contiguous() || (wpe && !wpe->contiguous()))
        throw KernelError("embed_bigram: tables of one type and width, bigram [buckets + 1, width], a float32 x and an int32 state expected");
    static auto fn = SANDY_KERNEL(streams, sandy_embed_bigram);
    static auto keep = SANDY_KERNEL(streams, sandy_bigram_keep);
    {
        OpTimer timer(l, "embedding", (double)s.n_tokens * x.cols * (3.0 * wte.elem_size() + 4.0), 0);
        check(fn(ids, positions, s.token_seq, s.q_start, s.seq_slots, wte.data, bigram.data, wpe ? wpe->data : nullptr, b.buckets,
                 b.mul_prev, b.mul_cur, (int*)state.data, state.row_elems, (float*)x.data, (int)x.ld, s.n_tokens, (int)wte.rows,
                 wpe ? (int)wpe->rows : 0, (int)x.cols, code_of(wte.dtype), max_q_len <= 1 ? 1 : 0, l.status, l.stream),
              "embed_bigram");
    }
    if (max_q_len > 1) {
        OpTimer timer(l, "embedding: last tokens kept", 0, 0);
        check(keep(ids, s.q_start, s.seq_slots, (int*)state.data, state.row_elems, s.n_seqs, l.stream), "bigram_keep");
    }
}


void delta_scan(const Launch& l, const StepSeqs& s, const DeltaShape& d, const Tensor& qkv, const Tensor& bg, const StateView& state,
                Tensor& out, int max_q_len) {
    if (out.dtype != DType::F32 || out.cols != (int64_t)d.n_heads * d.v_dim || qkv.dtype != DType::F32)
        throw KernelError("delta_scan: float32 qkv and out [T, H * e] expected");
    static auto fn = SANDY_KERNEL(matrix_state, sandy_delta_scan);
    static auto chunked = SANDY_KERNEL(matrix_state, sandy_delta_chunk_scan);
    const int long_from = max_q_len >= kChunkedFrom ? kChunkedFrom : 0;
    const double st = 2.0 * s.n_seqs * d.n_heads * d.qk_dim * d.v_dim * 4.0;
    OpTimer timer(l, "delta rule: recurrence", st + tensor_bytes(&qkv) + tensor_bytes(&out), 6.0 * s.n_tokens * d.n_heads * d.qk_dim * d.v_dim);
    const std::string shape = "(d=" + std::to_string(d.qk_dim) + ",e=" + std::to_string(d.v_dim) + ")";
    check(fn((const float*)qkv.data, (int)qkv.ld, (const float*)bg.data, (float*)state.data, state.row_elems, s.q_start, s.seq_slots,
             (float*)out.data, (int)out.ld, s.n_seqs, d.n_heads, d.n_qk_heads, d.qk_dim, d.v_dim, long_from, l.stream),
          "delta_scan" + shape);
    if (long_from)
        check(chunked((const float*)qkv.data, (int)qkv.ld, (const float*)bg.data, (float*)state.data, state.row_elems, s.q_start,
                      s.seq_slots, (float*)out.data, (int)out.ld, s.n_seqs, d.n_heads, d.n_qk_heads, d.qk_dim, d.v_dim, long_from,
                      l.stream),
              "delta_chunk_scan" + shape);
}

void mlstm_scan(const Launch& l, const StepSeqs& s, const MlstmShape& m, const Tensor& proj, const Tensor& gates,
                const float* gate_bias, const StateView& state, Tensor& out, int max_q_len) {
    if (out.dtype != DType::F32 || out.cols != (int64_t)m.n_heads * m.v_dim || gates.dtype != DType::F32 || gates.cols < 2 * m.n_heads ||
        state.dtype != DType::F32 || state.row_elems < mlstm_state_floats(m.n_heads, m.qk_dim, m.v_dim))
        throw KernelError("mlstm_scan: shapes disagree");
    static auto fn = SANDY_KERNEL(matrix_state, sandy_mlstm_scan);
    static auto chunked = SANDY_KERNEL(matrix_state, sandy_mlstm_chunk_scan);
    const int long_from = max_q_len >= kChunkedFrom ? kChunkedFrom : 0;
    const double st = 2.0 * s.n_seqs * m.n_heads * m.qk_dim * m.v_dim * 4.0;
    OpTimer timer(l, "matrix memory: recurrence", st + tensor_bytes(&out), 4.0 * s.n_tokens * m.n_heads * m.qk_dim * m.v_dim);
    const std::string shape = "(d=" + std::to_string(m.qk_dim) + ",e=" + std::to_string(m.v_dim) + ")";
    check(fn(proj.data, (int)proj.ld, code_of(proj.dtype), m.q_off, m.k_off, m.v_off, (const float*)gates.data, (int)gates.ld, gate_bias,
             m.cap, m.q_scale, (float*)state.data, state.row_elems, s.q_start, s.seq_slots, (float*)out.data, (int)out.ld, s.n_seqs,
             m.n_heads, m.qk_dim, m.v_dim, long_from, l.stream),
          "mlstm_scan" + shape);
    if (long_from)
        check(chunked(proj.data, (int)proj.ld, code_of(proj.dtype), m.q_off, m.k_off, m.v_off, (const float*)gates.data, (int)gates.ld,
                      gate_bias, m.cap, m.q_scale, (float*)state.data, state.row_elems, s.q_start, s.seq_slots, (float*)out.data,
                      (int)out.ld, s.n_seqs, m.n_heads, m.qk_dim, m.v_dim, long_from, l.stream),
              "mlstm_chunk_scan" + shape);
}

void sample(const Launch& l, const Tensor& logits, int* out_tokens, const float* temperature, const int* top_k,
            const float* top_p, const float* uniform, const SampleFeedback* fb) {
    if (logits.dtype != DType::F32) throw KernelError("sample: logits must be float32");
    if (temperature && !uniform) throw KernelError("sample: temperature sampling needs a uniform number per row");
    static auto fn = SANDY_KERNEL(sampling, sandy_sample);
    OpTimer timer(l, "sampling", tensor_bytes(&logits), 0);
    check(fn((const float*)logits.data, (int)logits.ld, (int)logits.rows, (int)logits.cols, temperature, top_k, top_p, uniform,
             out_tokens, l.status, fb ? fb->token_ids : nullptr, fb ? fb->logit_rows : nullptr, fb ? fb->positions : nullptr,
             fb ? fb->burst_tokens : nullptr, fb ? fb->row_step : nullptr, l.stream),
          "sample");
}

}  // namespace ops
}  // namespace sandy
