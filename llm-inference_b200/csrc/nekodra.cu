// Model family "Nekodra": a decoder of parallel layers, x <- x + (mixer(LN1(x)) + ff(LN2(x))), whose mixer is latent
// attention without positions (one cached low-rank row per token, a softmax sink per head, a sigmoid output gate,
// optional reuse of an earlier layer's cached rows) and whose feed-forward is a routed mixture of GLU experts with
// identity experts and a shared expert. Learned absolute positions are added to the embedding; layer norms carry
// weight and bias. Everything config.json gives is read per layer; nothing is assumed equal across layers.
//
// A step runs on the family-independent pieces of the library: SequenceBatch / PagePool for slots and pages,
// b200_layernorm_pair, b200_gemm_grouped (dense, per-head strided, and per-expert grouped products), the latent
// attention kernels and the MoE kernels. The residual stream, norms, softmax and router are fp32 in both serving
// dtypes; in B200_BF16 the GEMM operands (weights, normed activations, cached rows) are bfloat16.
//
// Launch order per layer (T tokens of all entries packed; H heads, dq / dv per-head sizes, R latent rank):
//   LN pair -> [q | gate | down-projected row] = h1 W_in^T (one GEMM) -> RMS norm + page store of the row
//   -> qa_h = W_uk,h^T q_h (strided batch over heads) -> latent attention over the pages -> a_h = (W_uv,h o_h) *
//   sigmoid(gate_h) (strided batch, gate in the epilogue) -> W_o;   router -> counting sort -> grouped GLU GEMM ->
//   grouped down GEMM;   shared GLU GEMM -> down GEMM;   x += mixer + routed + shared (one kernel).
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "launch_count.h"
#include "model_registry.h"
#include "checkpoint_upload.h"
#include "safetensors.h"

namespace b200 {
namespace {

constexpr int kPageRows = 64;

struct NkLayer {
    int heads = 0, dq = 0, dv = 0, rank = 0, kv_from = -1, cache = -1;   // cache: index of the pool this layer reads
    bool owns_cache = false;
    float scale = 1.f;
    int n_in = 0;   // rows of w_in: H*dq + H*dv (+ rank when the layer projects its own rows)
    float *n1w = nullptr, *n1b = nullptr, *n2w = nullptr, *n2b = nullptr, *dkv_norm = nullptr, *sink = nullptr;
    void *w_in = nullptr, *uk = nullptr, *uv = nullptr, *o = nullptr;
    // feed-forward
    bool has_mlp = false;
    int experts = 0, identity = 0, top = 0, ff = 0, shared_ff = 0;
    float route_scale = 1.f;
    float *router = nullptr, *correction = nullptr;
    void *w_gu = nullptr, *w_down = nullptr, *s_gu = nullptr, *s_down = nullptr;
};

class Nekodra : public Model {
public:
    ~Nekodra() override {
        if (stream_) cudaStreamSynchronize(stream_);
        for (void* p : owned_) cudaFree(p);
        cudaFree(scratch_);
        cudaFree(ws_);
        cudaFree(attn_ws_);
        cudaFree(capture_);
        if (logits_host_) cudaFreeHost(logits_host_);
        if (stream_) cudaStreamDestroy(stream_);
    }
    const char* family() const override { return "Nekodra"; }
    int vocab() const override { return vocab_; }
    int width() const override { return D_; }
    int layer_count() const override { return (int)layers_.size(); }
    int n_slots() const override { return seq_.n_slots; }
    int max_positions() const override { return seq_.max_positions; }
    int page_rows() const override { return seq_.pool.page_rows(); }
    int pages_total() const override { return seq_.pool.n_pages(); }
    int pages_free() const override { return seq_.pool.free_count(); }
    int slot_length(int slot) const override { return seq_.length[slot]; }
    int slot_page_count(int slot) const override { return seq_.pool.owned(slot); }
    int slot_pages(int slot, int* out, int max_n) const override {
        const int n = std::min(max_n, seq_.pool.owned(slot));
        for (int i = 0; i < n; ++i) out[i] = seq_.pool.list(slot)[i];
        return n;
    }
    int step_launches() const override { return launches_; }

    int load(const ModelDir& dir, const b200_model_options& opt, std::string& err);
    int step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) override;
    int release(int slot) override {
        cudaStreamSynchronize(stream_);   // pages change owner only behind the work that reads them
        return seq_.release(slot);
    }
    int capture_layers(int on) override { capture_on_ = on != 0; return B200_OK; }
    int captured_layers(float* out, size_t max_floats) override {
        const size_t n = (size_t)layers_.size() * captured_tokens_ * D_;
        if (!capture_ || n == 0) return 0;
        if (n > max_floats) return B200_EWORKSPACE;
        cudaStreamSynchronize(stream_);
        if (cudaMemcpy(out, capture_, n * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return B200_EINVAL;
        return captured_tokens_;
    }

private:
    size_t esz() const { return dtype_ == B200_BF16 ? 2 : 4; }
    // checkpoint tensor -> device, converted to the serving dtype (or fp32 when as_f32); rows of several tensors can be
    // stacked into one device matrix by passing the destination
    int upload(const SafeTensorsFile& st, const std::string& name, std::vector<long long> shape, bool as_f32, void* dst,
               std::string& err);
    void* dalloc(size_t bytes) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) return nullptr;
        owned_.push_back(p);
        return p;
    }
    int gemm(const void* A, int a_dt, long long lda, const void* W, long long ldw, void* C, int c_dt, long long ldc, int M, int N,
             int K, int epi = B200_GG_NONE, const float* aux = nullptr, long long ld_aux = 0);
    int ensure_scratch(int T, int W);

    int dtype_ = B200_BF16, vocab_ = 0, D_ = 0;
    float eps_ = 1e-5f;
    std::vector<NkLayer> layers_;
    void *embed_ = nullptr, *pos_ = nullptr, *head_ = nullptr;
    float *fnw_ = nullptr, *fnb_ = nullptr;
    std::vector<void*> pools_;   // one latent pool per cache-owning layer: [n_pages, kPageRows, rank]
    SequenceBatch seq_;
    std::vector<void*> owned_;
    cudaStream_t stream_ = nullptr;
    // scratch, grown to the largest step seen
    char* scratch_ = nullptr;
    void* ws_ = nullptr;          // split-K partials of the weight-streaming GEMM
    size_t ws_bytes_ = 0;
    void* attn_ws_ = nullptr;     // shares of split-context attention (decode batches)
    size_t attn_ws_bytes_ = 0;
    int cap_T_ = 0, cap_W_ = 0;
    float *x_ = nullptr, *proj_ = nullptr, *qa_ = nullptr, *oa_ = nullptr, *mix_ = nullptr, *eo_ = nullptr, *sh_ = nullptr,
          *weight_ = nullptr, *logits_ = nullptr;
    void *h1_ = nullptr, *h2_ = nullptr, *att_ = nullptr, *act_ = nullptr, *sact_ = nullptr, *hf_ = nullptr;
    int *chosen_ = nullptr, *group_off_ = nullptr, *src_row_ = nullptr, *dest_ = nullptr, *ids_dev_ = nullptr;
    float* logits_host_ = nullptr;
    size_t logits_host_floats_ = 0;
    // sizes the scratch depends on (maxima over layers)
    int max_in_ = 0, max_hr_ = 0, max_hdv_ = 0, max_top_ = 0, max_ff_ = 0, max_sff_ = 0, max_experts_ = 0;
    bool capture_on_ = false;
    float* capture_ = nullptr;
    int capture_cap_ = 0, captured_tokens_ = 0;
    int launches_ = 0;
};

int Nekodra::upload(const SafeTensorsFile& st, const std::string& name, std::vector<long long> shape, bool as_f32, void* dst,
                    std::string& err) {
    return upload_tensor(st, name, shape, as_f32, dtype_, dst, err);
}

#define NK_TRY(call)                    \
    do {                                \
        const int rc_ = (call);         \
        if (rc_ != B200_OK) return rc_; \
    } while (0)

int Nekodra::load(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    const Json& c = dir.config;
    dtype_ = opt.dtype;
    if (dtype_ != B200_BF16 && dtype_ != B200_F32) { err = "dtype must be bfloat16 or float32"; return B200_EINVAL; }
    vocab_ = (int)c.integer("vocab", 0);
    D_ = (int)c.integer("width", 0);
    const int max_pos = (int)c.integer("max_positions", 0);
    const Json* norm = c.get("norm");
    eps_ = norm ? (float)norm->number("eps", 1e-5) : 1e-5f;
    const Json* ls = c.get("layers");
    if (vocab_ < 1 || D_ < 1 || max_pos < 1 || !norm || !ls || ls->kind != Json::Arr || ls->arr.empty()) {
        err = "config.json: vocab, width, max_positions, norm.eps and layers are required";
        return B200_EINVAL;
    }
    if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) { err = "no CUDA device: this library has no CPU path"; return B200_EINVAL; }
    SafeTensorsFile st;
    if (!st.open(dir.path + "/model.safetensors", err)) return B200_EINVAL;
    NK_TRY(seq_.init(opt.max_tokens, kPageRows, opt.max_slots, max_pos, err));

    const size_t E = esz();
    const long long D = D_;
    auto f32 = [&](const std::string& name, long long n, float*& dst) -> int {
        dst = (float*)dalloc((size_t)n * 4);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload(st, name, {n}, true, dst, err);
    };
    auto mat = [&](const std::string& name, long long rows, long long cols, void*& dst) -> int {
        dst = dalloc((size_t)rows * cols * E);
        if (!dst) { err = "out of device memory"; return B200_ENOMEM; }
        return upload(st, name, {rows, cols}, false, dst, err);
    };
    NK_TRY(mat("embed", vocab_, D, embed_));
    NK_TRY(mat("pos", max_pos, D, pos_));
    NK_TRY(mat("head", vocab_, D, head_));
    NK_TRY(f32("final.norm", D, fnw_));
    NK_TRY(f32("final.norm.b", D, fnb_));

    layers_.resize(ls->arr.size());
    for (size_t i = 0; i < layers_.size(); ++i) {
        const Json& lj = ls->arr[i];
        NkLayer& L = layers_[i];
        const std::string pre = "l" + std::to_string(i) + ".";
        const std::string type = lj.text("type");
        if (type != "latent_attention") { err = "layer " + std::to_string(i) + ": mixer type '" + type + "' is not part of this family"; return B200_EUNSUPPORTED; }
        const Json* mx = lj.get("mixer");
        if (!mx) { err = "layer " + std::to_string(i) + ": no mixer"; return B200_EINVAL; }
        L.heads = (int)mx->integer("heads", 0);
        L.dq = (int)mx->integer("dim", 0);
        L.dv = (int)mx->integer("vdim", 0);
        L.rank = (int)mx->integer("kv_rank", 0);
        L.scale = (float)mx->number("scale", 0.0);
        if (L.heads < 1 || L.dq < 1 || L.dv < 1 || L.rank < 1 || !mx->has("scale")) { err = "layer " + std::to_string(i) + ": mixer needs heads, dim, vdim, kv_rank, scale"; return B200_EINVAL; }
        if (L.rank > 512) { err = "kv_rank above 512 is not supported by the latent attention kernels"; return B200_EUNSUPPORTED; }
        if (mx->has("kv_from")) {
            L.kv_from = (int)mx->integer("kv_from", -1);
            if (L.kv_from < 0 || L.kv_from >= (int)i || !layers_[L.kv_from].owns_cache || layers_[L.kv_from].rank != L.rank) {
                err = "layer " + std::to_string(i) + ": kv_from must name an earlier layer that projects its own rows of the same kv_rank";
                return B200_EINVAL;
            }
            L.cache = layers_[L.kv_from].cache;
        } else {
            L.owns_cache = true;
            L.cache = (int)pools_.size();
            void* pool = dalloc((size_t)seq_.pool.n_pages() * kPageRows * L.rank * E);
            if (!pool) { err = "out of device memory (latent cache)"; return B200_ENOMEM; }
            cudaMemset(pool, 0, (size_t)seq_.pool.n_pages() * kPageRows * L.rank * E);
            pools_.push_back(pool);
        }
        const long long nq = (long long)L.heads * L.dq, ng = (long long)L.heads * L.dv;
        L.n_in = (int)(nq + ng + (L.owns_cache ? L.rank : 0));
        NK_TRY(f32(pre + "norm1", D, L.n1w));
        NK_TRY(f32(pre + "norm1.b", D, L.n1b));
        NK_TRY(f32(pre + "norm2", D, L.n2w));
        NK_TRY(f32(pre + "norm2.b", D, L.n2b));
        NK_TRY(f32(pre + "mix.sink", L.heads, L.sink));
        // one input matrix: query rows, gate rows, then the down projection (all read the same normed input)
        L.w_in = dalloc((size_t)L.n_in * D * E);
        if (!L.w_in) { err = "out of device memory"; return B200_ENOMEM; }
        NK_TRY(upload(st, pre + "mix.q", {nq, D}, false, L.w_in, err));
        NK_TRY(upload(st, pre + "mix.g", {ng, D}, false, (char*)L.w_in + (size_t)nq * D * E, err));
        if (L.owns_cache) {
            NK_TRY(upload(st, pre + "mix.dkv", {L.rank, D}, false, (char*)L.w_in + (size_t)(nq + ng) * D * E, err));
            NK_TRY(f32(pre + "mix.dkv.norm", L.rank, L.dkv_norm));
        }
        NK_TRY(mat(pre + "mix.uk", nq, L.rank, L.uk));
        NK_TRY(mat(pre + "mix.uv", ng, L.rank, L.uv));
        NK_TRY(mat(pre + "mix.o", D, ng, L.o));
        max_in_ = std::max(max_in_, L.n_in);
        max_hr_ = std::max(max_hr_, L.heads * L.rank);
        max_hdv_ = std::max(max_hdv_, (int)ng);

        const Json* ml = lj.get("mlp");
        if (ml && !ml->is_null()) {
            const std::string kind = ml->text("kind");
            if (kind != "moe") { err = "layer " + std::to_string(i) + ": feed-forward kind '" + kind + "' is not part of this family"; return B200_EUNSUPPORTED; }
            const Json* r = ml->get("router");
            const Json* ex = ml->get("expert");
            if (!r) { err = "layer " + std::to_string(i) + ": mlp.router is required"; return B200_EINVAL; }
            L.has_mlp = true;
            L.experts = (int)r->integer("experts", 0);
            L.identity = (int)r->integer("identity", 0);
            L.top = (int)r->integer("top", 0);
            L.route_scale = (float)r->number("scale", 1.0);
            L.ff = ex ? (int)ex->integer("ff", 0) : 0;
            const int n_out = L.experts + L.identity;
            if (L.experts < 0 || L.identity < 0 || n_out < 1 || L.top < 1 || L.top > n_out || (L.experts > 0 && L.ff < 1)) {
                err = "layer " + std::to_string(i) + ": bad router / expert sizes";
                return B200_EINVAL;
            }
            L.router = (float*)dalloc((size_t)n_out * D * 4);
            if (!L.router) { err = "out of device memory"; return B200_ENOMEM; }
            NK_TRY(upload(st, pre + "mlp.router", {n_out, D}, true, L.router, err));
            NK_TRY(f32(pre + "mlp.correction", n_out, L.correction));
            if (L.experts > 0) {
                L.w_gu = dalloc((size_t)L.experts * 2 * L.ff * D * E);
                L.w_down = dalloc((size_t)L.experts * D * L.ff * E);
                if (!L.w_gu || !L.w_down) { err = "out of device memory"; return B200_ENOMEM; }
                for (int e = 0; e < L.experts; ++e) {
                    const std::string ep = pre + "mlp.e" + std::to_string(e) + ".";
                    char* gu = (char*)L.w_gu + (size_t)e * 2 * L.ff * D * E;
                    NK_TRY(upload(st, ep + "gate", {L.ff, D}, false, gu, err));
                    NK_TRY(upload(st, ep + "up", {L.ff, D}, false, gu + (size_t)L.ff * D * E, err));
                    NK_TRY(upload(st, ep + "down", {D, L.ff}, false, (char*)L.w_down + (size_t)e * D * L.ff * E, err));
                }
            }
            const Json* sh = ml->get("shared");
            if (sh && !sh->is_null()) {
                L.shared_ff = (int)sh->integer("ff", 0);
                if (L.shared_ff < 1) { err = "layer " + std::to_string(i) + ": mlp.shared.ff is required"; return B200_EINVAL; }
                L.s_gu = dalloc((size_t)2 * L.shared_ff * D * E);
                if (!L.s_gu) { err = "out of device memory"; return B200_ENOMEM; }
                NK_TRY(upload(st, pre + "mlp.shared.gate", {L.shared_ff, D}, false, L.s_gu, err));
                NK_TRY(upload(st, pre + "mlp.shared.up", {L.shared_ff, D}, false, (char*)L.s_gu + (size_t)L.shared_ff * D * E, err));
                NK_TRY(mat(pre + "mlp.shared.down", D, L.shared_ff, L.s_down));
            }
            max_top_ = std::max(max_top_, L.top);
            max_ff_ = std::max(max_ff_, L.ff);
            max_sff_ = std::max(max_sff_, L.shared_ff);
            max_experts_ = std::max(max_experts_, L.experts);
        }
    }
    if (cudaDeviceSynchronize() != cudaSuccess) { err = "weight upload failed"; return B200_EINVAL; }
    return B200_OK;
}

int Nekodra::ensure_scratch(int T, int W) {
    if (T <= cap_T_ && W <= cap_W_) return B200_OK;
    const int cT = std::max(T, cap_T_), cW = std::max(W, cap_W_);
    cudaStreamSynchronize(stream_);
    cudaFree(scratch_);
    scratch_ = nullptr;
    cap_T_ = cap_W_ = 0;
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t E = esz(), t = (size_t)cT, top = (size_t)std::max(1, max_top_);
    const size_t sizes[] = {
        al(t * D_ * 4),                 // x
        al(t * max_in_ * 4),            // proj
        al(t * max_hr_ * 4),            // qa
        al(t * max_hr_ * 4),            // oa
        al(t * D_ * 4),                 // mix
        al(t * top * D_ * 4),           // eo
        al(t * D_ * 4),                 // sh
        al(t * top * 4),                // weight
        al((size_t)cW * vocab_ * 4),    // logits
        al(t * D_ * E),                 // h1
        al(t * D_ * E),                 // h2
        al(t * max_hdv_ * E),           // att
        al(t * top * std::max(1, max_ff_) * E),   // act
        al(t * std::max(1, max_sff_) * E),        // sact
        al((size_t)cW * D_ * E),        // hf
        al(t * top * 4),                // chosen
        al((size_t)(max_experts_ + 2) * 4),       // group_off
        al(t * top * 4),                // src_row
        al(t * top * 4),                // dest
        al((size_t)cW * 4),             // ids
    };
    size_t total = 0;
    for (size_t s : sizes) total += s;
    if (cudaMalloc(&scratch_, total) != cudaSuccess) return B200_ENOMEM;
    char* p = scratch_;
    int k = 0;
    auto take = [&](auto*& dst) { dst = reinterpret_cast<std::remove_reference_t<decltype(dst)>>(p); p += sizes[k++]; };
    take(x_); take(proj_); take(qa_); take(oa_); take(mix_); take(eo_); take(sh_); take(weight_); take(logits_);
    take(h1_); take(h2_); take(att_); take(act_); take(sact_); take(hf_);
    take(chosen_); take(group_off_); take(src_row_); take(dest_); take(ids_dev_);
    cap_T_ = cT;
    cap_W_ = cW;
    const size_t lf = (size_t)cW * vocab_;
    if (lf > logits_host_floats_) {
        if (logits_host_) cudaFreeHost(logits_host_);
        logits_host_ = nullptr;
        if (cudaMallocHost(&logits_host_, lf * 4) != cudaSuccess) return B200_ENOMEM;
        logits_host_floats_ = lf;
    }
    return B200_OK;
}

int Nekodra::gemm(const void* A, int a_dt, long long lda, const void* W, long long ldw, void* C, int c_dt, long long ldc, int M,
                  int N, int K, int epi, const float* aux, long long ld_aux) {
    if (lda == K && ldw == K && ldc == N && !aux && a_dt == dtype_) {   // contiguous: the tcgen05 GEMM when it fits
        const size_t need = b200_linear_ex_workspace_bytes(M, N, K);
        if (need > ws_bytes_) {
            cudaStreamSynchronize(stream_);
            cudaFree(ws_);
            ws_ = nullptr;
            ws_bytes_ = 0;
            if (cudaMalloc(&ws_, need) == cudaSuccess) ws_bytes_ = need;   // without it the call runs with a single split
        }
        return b200_linear_ex(A, W, C, M, N, K, a_dt, c_dt, epi, ws_, ws_bytes_, stream_);
    }
    b200_gemm_grouped_args g{};
    g.A = A; g.W = W; g.C = C; g.aux = aux;
    g.lda = lda; g.ldw = ldw; g.ldc = ldc; g.ld_aux = ld_aux;
    g.M = M; g.N = N; g.K = K; g.batch = 1; g.trans_b = 1; g.epi = epi;
    g.a_dtype = a_dt; g.w_dtype = dtype_; g.c_dtype = c_dt;
    return b200_gemm_grouped(&g, stream_);
}

int Nekodra::step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) {
    if (entries.empty()) return B200_OK;
    const uint64_t launches0 = b200_launch_count();
    NK_TRY(seq_.begin_step(entries, stream_, err));
    const int T = seq_.n_tokens, W = seq_.n_want, D = D_, dt = dtype_;
    if (ensure_scratch(T, std::max(W, 1)) != B200_OK) { err = "step: out of device memory for the scratch buffers"; return B200_ENOMEM; }
    int longest_entry = 0, longest_context = 0;
    for (const StepEntry& en : entries) {
        longest_entry = std::max(longest_entry, en.n_tokens);
        longest_context = std::max(longest_context, seq_.length[en.slot]);
    }
    if (longest_entry == 1) {   // a decode batch: room for the shares of split contexts
        size_t need = 0;
        for (const NkLayer& L : layers_) need = std::max(need, b200_latent_attention_workspace_bytes(T, L.heads, L.rank));
        if (need > attn_ws_bytes_) {
            cudaStreamSynchronize(stream_);
            cudaFree(attn_ws_);
            attn_ws_ = nullptr;
            attn_ws_bytes_ = 0;
            if (cudaMalloc(&attn_ws_, need) == cudaSuccess) attn_ws_bytes_ = need;
        }
    }
    const int* pages = seq_.pool.device();
    const int max_pages = seq_.pool.max_pages();
    if (capture_on_) {
        const size_t need = (size_t)layers_.size() * T * D;
        if ((size_t)capture_cap_ < need) {
            cudaStreamSynchronize(stream_);
            cudaFree(capture_);
            capture_ = nullptr;
            if (cudaMalloc(&capture_, need * 4) != cudaSuccess) { err = "step: no memory to keep the layers"; return B200_ENOMEM; }
            capture_cap_ = (int)need;
        }
        captured_tokens_ = T;
    }
#define NK_OP(call)                                                             \
    do {                                                                        \
        const int rc_ = (call);                                                 \
        if (rc_ != B200_OK) { err = std::string(#call) + " failed (" + std::to_string(rc_) + ")"; return rc_; } \
    } while (0)
    NK_OP(b200_embed_positions(seq_.d_ids(), seq_.d_pos(), embed_, pos_, x_, T, D, dt, stream_));
    for (size_t li = 0; li < layers_.size(); ++li) {
        const NkLayer& L = layers_[li];
        const int H = L.heads, R = L.rank, nq = H * L.dq, ng = H * L.dv;
        NK_OP(b200_layernorm_pair(x_, nullptr, T, D, eps_, L.n1w, L.n1b, h1_, L.has_mlp ? L.n2w : nullptr, L.has_mlp ? L.n2b : nullptr,
                                  L.has_mlp ? h2_ : nullptr, dt, stream_));
        // ---- mixer
        NK_OP(gemm(h1_, dt, D, L.w_in, D, proj_, B200_F32, L.n_in, T, L.n_in, D));
        if (L.owns_cache)
            NK_OP(b200_latent_store(proj_ + nq + ng, L.n_in, L.dkv_norm, eps_, pools_[L.cache], pages, max_pages, kPageRows,
                                    seq_.d_slot(), seq_.d_pos(), T, R, dt, stream_));
        {   // qa[t, h, :] = sum_d q[t, h, d] W_uk[h*dq + d, :]
            b200_gemm_grouped_args g{};
            g.A = proj_; g.lda = L.n_in; g.stride_a = L.dq;
            g.W = L.uk; g.ldw = R; g.stride_w = (long long)L.dq * R; g.trans_b = 0;
            g.C = qa_; g.ldc = (long long)H * R; g.stride_c = R;
            g.M = T; g.N = R; g.K = L.dq; g.batch = H;
            g.a_dtype = B200_F32; g.w_dtype = dt; g.c_dtype = B200_F32;
            NK_OP(b200_gemm_grouped(&g, stream_));
        }
        NK_OP(b200_latent_attention(qa_, oa_, pools_[L.cache], pages, max_pages, kPageRows, seq_.d_slot(), seq_.d_pos(), L.sink,
                                    L.scale, T, H, R, dt, longest_entry, longest_context, attn_ws_, attn_ws_bytes_, stream_));
        {   // att[t, h, :] = (W_uv,h oa[t, h, :]) * sigmoid(gate[t, h, :])
            b200_gemm_grouped_args g{};
            g.A = oa_; g.lda = (long long)H * R; g.stride_a = R;
            g.W = L.uv; g.ldw = R; g.stride_w = (long long)L.dv * R; g.trans_b = 1;
            g.C = att_; g.ldc = ng; g.stride_c = L.dv;
            g.aux = proj_ + nq; g.ld_aux = L.n_in; g.stride_aux = L.dv; g.epi = B200_GG_SIGMOID_MUL;
            g.M = T; g.N = L.dv; g.K = R; g.batch = H;
            g.a_dtype = B200_F32; g.w_dtype = dt; g.c_dtype = dt;
            NK_OP(b200_gemm_grouped(&g, stream_));
        }
        NK_OP(gemm(att_, dt, ng, L.o, ng, mix_, B200_F32, D, T, D, ng));
        // ---- feed-forward
        const bool routed = L.has_mlp;
        if (L.has_mlp) {
            NK_OP(b200_moe_route(h2_, dt, L.router, L.correction, T, D, L.experts + L.identity, L.top, L.route_scale, chosen_, weight_,
                                 stream_));
            NK_OP(b200_moe_dispatch(chosen_, T, L.top, L.experts, group_off_, src_row_, dest_, stream_));
            if (L.experts > 0) {
                b200_gemm_grouped_args g{};
                g.A = h2_; g.lda = D; g.a_rows = src_row_; g.group_off = group_off_;
                g.W = L.w_gu; g.ldw = D; g.stride_w = (long long)2 * L.ff * D; g.trans_b = 1; g.epi = B200_GG_GLU;
                g.C = act_; g.ldc = L.ff;
                g.M = T; g.N = L.ff; g.K = D; g.batch = L.experts;   // an expert owns at most one row per token
                g.a_dtype = dt; g.w_dtype = dt; g.c_dtype = dt;
                NK_OP(b200_gemm_grouped(&g, stream_));
                b200_gemm_grouped_args d{};
                d.A = act_; d.lda = L.ff; d.group_off = group_off_;
                d.W = L.w_down; d.ldw = L.ff; d.stride_w = (long long)D * L.ff; d.trans_b = 1;
                d.C = eo_; d.ldc = D;
                d.M = T; d.N = D; d.K = L.ff; d.batch = L.experts;
                d.a_dtype = dt; d.w_dtype = dt; d.c_dtype = B200_F32;
                NK_OP(b200_gemm_grouped(&d, stream_));
            }
            if (L.shared_ff > 0) {
                NK_OP(gemm(h2_, dt, D, L.s_gu, D, sact_, dt, L.shared_ff, T, L.shared_ff, D, B200_GG_GLU));
                NK_OP(gemm(sact_, dt, L.shared_ff, L.s_down, L.shared_ff, sh_, B200_F32, D, T, D, L.shared_ff));
            }
        }
        NK_OP(b200_residual_combine(x_, mix_, L.has_mlp && L.shared_ff > 0 ? sh_ : nullptr, eo_, routed ? dest_ : nullptr, weight_, h2_, dt,
                                    T, D, L.top, stream_));
        if (capture_on_)
            cudaMemcpyAsync(capture_ + li * (size_t)T * D, x_, (size_t)T * D * 4, cudaMemcpyDeviceToDevice, stream_);
    }
    if (W > 0) {
        NK_OP(b200_layernorm_pair(x_, seq_.d_want_rows(), W, D, eps_, fnw_, fnb_, hf_, nullptr, nullptr, nullptr, dt, stream_));
        NK_OP(gemm(hf_, dt, D, head_, D, logits_, B200_F32, vocab_, W, vocab_, D));
        if (ids_out) NK_OP(b200_argmax(logits_, ids_dev_, W, vocab_, B200_F32, stream_));
        if (logits_out) cudaMemcpyAsync(logits_host_, logits_, (size_t)W * vocab_ * 4, cudaMemcpyDeviceToHost, stream_);
        if (ids_out) cudaMemcpyAsync(ids_out, ids_dev_, (size_t)W * 4, cudaMemcpyDeviceToHost, stream_);
    }
    const cudaError_t e = cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) { err = std::string("step: ") + cudaGetErrorString(e); return (int)e; }
    if (W > 0 && logits_out) memcpy(logits_out, logits_host_, (size_t)W * vocab_ * 4);
    launches_ = (int)(b200_launch_count() - launches0);
    return B200_OK;
#undef NK_OP
}

Model* make_nekodra(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    Nekodra* m = new Nekodra();
    if (m->load(dir, opt, err) != B200_OK) {
        delete m;
        return nullptr;
    }
    return m;
}

FamilyRegistrar reg_nekodra("Nekodra", make_nekodra);

}  // namespace
}  // namespace b200
