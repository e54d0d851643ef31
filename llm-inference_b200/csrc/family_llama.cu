// Model family "llama": the LLaMA engine (b200_engine.h) behind the Model interface of the registry, so that LLaMA
// checkpoints are opened, scheduled and sampled through the same entry points as every other family (b200_model_open,
// b200_model_step, b200_model_generate, bin/b200_serve).
//
// Folder layout: config.json {"architecture": "llama", "num_layers", "head_num", "kv_head_num", "head_size", "inter_size",
// "vocab_size", "max_seq_len", "rms_eps", "rotary_dim", "rotary_base"} next to the reference's raw weight files
// (b200_engine_load_weights; llama_weights.cc:41-53). "random_init": {"seed", "std"} instead of weight files gives a
// random model (benches, tests). fp16 only: a step is the engine's ragged prompt pass (b200_engine_prefill_ragged: every
// entry's tokens appended behind that slot's history, slots without an entry sit the pass out), which yields the logits
// and the greedy pick of each entry's LAST token; other wanted places are refused. The cache is the engine's paged KV
// cache (pages of 128 rows from the shared PagePool) when head size and head ratio allow it, else its dense cache.
#include <algorithm>
#include <cstring>

#include "b200_engine.h"
#include "common.cuh"
#include "model_registry.h"

namespace b200 {
namespace {

__global__ void half_rows_to_float_kernel(const __half* __restrict__ src, float* __restrict__ dst, const int* __restrict__ rows, int vocab) {
    const __half* s = src + (size_t)rows[blockIdx.x] * vocab;
    float* d = dst + (size_t)blockIdx.x * vocab;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) d[i] = __half2float(s[i]);
}

class LlamaFamily : public Model {
public:
    ~LlamaFamily() override {
        if (eng_) b200_engine_destroy(eng_);
        cudaFree(rows_dev_);
        cudaFree(logits_f32_);
    }
    const char* family() const override { return "llama"; }
    int vocab() const override { return cfg_.vocab_size; }
    int width() const override { return cfg_.head_num * cfg_.head_size; }
    int layer_count() const override { return cfg_.num_layers; }
    int n_slots() const override { return slots_; }
    int max_positions() const override { return cfg_.max_seq_len; }
    int page_rows() const override { return 128; }
    int pages_total() const override { return paged_ ? b200_engine_kv_pages_total(eng_) : slots_ * per_slot_pages(); }
    int pages_free() const override {
        if (paged_) return b200_engine_kv_pages_free(eng_);
        int used = 0;
        for (int b = 0; b < slots_; ++b) used += slot_page_count(b);
        return pages_total() - used;
    }
    int slot_length(int slot) const override { return length_[slot]; }
    int slot_page_count(int slot) const override { return (length_[slot] + 127) / 128; }
    int slot_pages(int, int*, int) const override { return 0; }   // the engine keeps its lists on the device side
    int step_launches() const override { return b200_engine_prefill_launches(eng_); }

    int load(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
        const Json& c = dir.config;
        memset(&cfg_, 0, sizeof cfg_);
        cfg_.num_layers = (int)c.integer("num_layers", 0);
        cfg_.head_num = (int)c.integer("head_num", 0);
        cfg_.kv_head_num = (int)c.integer("kv_head_num", cfg_.head_num);
        cfg_.head_size = (int)c.integer("head_size", 0);
        cfg_.inter_size = (int)c.integer("inter_size", 0);
        cfg_.vocab_size = (int)c.integer("vocab_size", 0);
        cfg_.max_seq_len = (int)c.integer("max_seq_len", 0);
        cfg_.rms_eps = (float)c.number("rms_eps", 1e-5);
        cfg_.rotary_dim = (int)c.integer("rotary_dim", cfg_.head_size);
        cfg_.rotary_base = (float)c.number("rotary_base", 10000.0);
        cfg_.dtype = B200_F16;
        cfg_.tp_size = 1;
        cfg_.max_batch = opt.max_slots;
        if (cfg_.num_layers < 1 || cfg_.head_num < 1 || cfg_.head_size < 1 || cfg_.inter_size < 1 || cfg_.vocab_size < 1 || cfg_.max_seq_len < 1) {
            err = "config.json: num_layers, head_num, head_size, inter_size, vocab_size and max_seq_len are required";
            return B200_EINVAL;
        }
        slots_ = opt.max_slots;
        const int g = cfg_.head_num / std::max(1, cfg_.kv_head_num);
        paged_ = cfg_.head_size == 128 && (g == 1 || g == 2 || g == 4 || g == 8) && cfg_.head_num % cfg_.kv_head_num == 0;
        const int n_pages = std::max(1, (opt.max_tokens + 127) / 128);
        eng_ = paged_ ? b200_engine_create_paged(&cfg_, slots_, B200_ENGINE_KV_PAGED, n_pages) : b200_engine_create_ex(&cfg_, slots_, 0);
        if (!eng_) { err = std::string("engine: ") + b200_engine_last_error(); return B200_EINVAL; }
        const Json* rnd = c.get("random_init");
        int rc;
        if (rnd && !rnd->is_null()) rc = b200_engine_init_random(eng_, (uint64_t)rnd->integer("seed", 1), (float)rnd->number("std", 0.02));
        else rc = b200_engine_load_weights(eng_, dir.path.c_str());
        if (rc != 0) { err = std::string("weights: ") + b200_engine_last_error(); return rc; }
        length_.assign(slots_, 0);
        if (cudaMalloc(&rows_dev_, (size_t)slots_ * sizeof(int)) != cudaSuccess ||
            cudaMalloc(&logits_f32_, (size_t)slots_ * cfg_.vocab_size * sizeof(float)) != cudaSuccess) { err = "out of device memory"; return B200_ENOMEM; }
        return B200_OK;
    }

    int step(const std::vector<StepEntry>& entries, float* logits_out, int* ids_out, std::string& err) override {
        if (entries.empty()) return B200_OK;
        std::vector<int> lens(slots_, 0), order(slots_, -1);
        for (size_t i = 0; i < entries.size(); ++i) {
            const StepEntry& en = entries[i];
            if (en.slot < 0 || en.slot >= slots_ || en.n_tokens < 1 || lens[en.slot]) { err = "step: bad slot or empty entry"; return B200_EINVAL; }
            if (en.n_want > 1 || (en.n_want == 1 && en.want[0] != en.n_tokens - 1)) {
                err = "llama: only the last place of an entry can be asked for";
                return B200_EUNSUPPORTED;
            }
            if (length_[en.slot] + en.n_tokens > cfg_.max_seq_len) { err = "step: sequence longer than max_seq_len"; return B200_EINVAL; }
            lens[en.slot] = en.n_tokens;
            order[en.slot] = (int)i;
        }
        std::vector<int> ids;   // packed in slot order, as the engine wants them
        for (int b = 0; b < slots_; ++b)
            if (order[b] >= 0) ids.insert(ids.end(), entries[order[b]].tokens, entries[order[b]].tokens + lens[b]);
        std::vector<int> picked(slots_, 0);
        const int rc = b200_engine_prefill_ragged(eng_, ids.data(), lens.data(), picked.data());
        if (rc != 0) { err = std::string("engine: ") + b200_engine_last_error(); return rc; }
        for (int b = 0; b < slots_; ++b) length_[b] += lens[b];
        std::vector<int> rows;
        for (const StepEntry& en : entries)
            if (en.n_want) rows.push_back(en.slot);
        if (ids_out)
            for (size_t k = 0; k < rows.size(); ++k) ids_out[k] = picked[rows[k]];
        if (logits_out && !rows.empty()) {
            cudaStream_t s = (cudaStream_t)b200_engine_stream(eng_);
            cudaMemcpyAsync(rows_dev_, rows.data(), rows.size() * sizeof(int), cudaMemcpyHostToDevice, s);
            half_rows_to_float_kernel<<<(unsigned)rows.size(), 256, 0, s>>>((const __half*)b200_engine_logits(eng_), logits_f32_, rows_dev_,
                                                                            cfg_.vocab_size);
            cudaMemcpyAsync(logits_out, logits_f32_, rows.size() * (size_t)cfg_.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, s);
            if (cudaStreamSynchronize(s) != cudaSuccess) { err = "step: logits copy failed"; return B200_EINVAL; }
        }
        return B200_OK;
    }
    int release(int slot) override {
        if (slot < 0 || slot >= slots_) return B200_EINVAL;
        length_[slot] = 0;
        return b200_engine_reset_slot(eng_, slot);
    }

private:
    int per_slot_pages() const { return (cfg_.max_seq_len + 127) / 128; }
    b200_model_config cfg_;
    b200_engine* eng_ = nullptr;
    int slots_ = 0;
    bool paged_ = false;
    std::vector<int> length_;
    int* rows_dev_ = nullptr;
    float* logits_f32_ = nullptr;
};

Model* make_llama(const ModelDir& dir, const b200_model_options& opt, std::string& err) {
    LlamaFamily* m = new LlamaFamily();
    if (m->load(dir, opt, err) != B200_OK) {
        delete m;
        return nullptr;
    }
    return m;
}

FamilyRegistrar reg_llama("llama", make_llama);

}  // namespace
}  // namespace b200
