// Page allocator of the paged caches (host side; kernels only ever read the lists).
// A pool of n_pages pages of page_rows rows each serves n_slots sequence slots; slot b owns the pages named by
// table[b * max_pages + 0 .. pages_of(b)), ONE list for all layers of a model (layer l uses the same page ids in its own
// pool). Entries of a living sequence's list are only ever APPENDED, so a queued list upload that runs late and picks
// up newer entries is harmless (kernels ahead of it never look past their own row count). Pages change owner only
// through release(), which callers run behind a stream synchronisation. Used by the LLaMA engine's paged KV cache
// (pages of 128 rows) and by the latent caches of the model families of b200_serve.h (pages of 64 rows).
#pragma once
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

namespace b200 {

class PagePool {
public:
    PagePool() = default;
    PagePool(const PagePool&) = delete;
    PagePool& operator=(const PagePool&) = delete;
    ~PagePool() { destroy(); }

    // extra_host_ints: room behind the pinned lists for the caller's own staging (e.g. per-slot row counts)
    cudaError_t init(int n_pages, int page_rows, int n_slots, int max_pages_per_slot, int extra_host_ints = 0) {
        destroy();
        n_pages_ = n_pages; page_rows_ = page_rows; n_slots_ = n_slots; max_pages_ = max_pages_per_slot;
        const size_t ints = (size_t)n_slots * max_pages_per_slot;
        cudaError_t e = cudaMalloc(&dev_, ints * sizeof(int));
        if (e != cudaSuccess) return e;
        if ((e = cudaMemset(dev_, 0, ints * sizeof(int))) != cudaSuccess) return e;
        if ((e = cudaMallocHost(&host_, (ints + extra_host_ints) * sizeof(int))) != cudaSuccess) return e;
        memset(host_, 0, (ints + extra_host_ints) * sizeof(int));
        owned_.assign(n_slots, 0);
        free_.resize(n_pages);
        for (int i = 0; i < n_pages; ++i) free_[i] = n_pages - 1 - i;   // page 0 is handed out first
        dirty_ = false;
        return cudaSuccess;
    }
    void destroy() {
        if (dev_) cudaFree(dev_);
        if (host_) cudaFreeHost(host_);
        dev_ = nullptr; host_ = nullptr;
        free_.clear(); owned_.clear();
    }
    bool ready() const { return dev_ != nullptr; }

    enum { kGrew = 1, kSame = 0, kTooLong = -1, kExhausted = -2 };
    // make sure slot b owns the pages of rows [0, rows)
    int ensure(int b, int rows) {
        const int need = (rows + page_rows_ - 1) / page_rows_;
        if (need > max_pages_) return kTooLong;
        if (need <= owned_[b]) return kSame;
        if ((size_t)(need - owned_[b]) > free_.size()) return kExhausted;
        int* list = host_ + (size_t)b * max_pages_;
        while (owned_[b] < need) {
            list[owned_[b]++] = free_.back();
            free_.pop_back();
        }
        dirty_ = true;
        return kGrew;
    }
    // pages that rows [0, rows) of slot b would still have to take
    int missing(int b, int rows) const {
        const int need = (rows + page_rows_ - 1) / page_rows_;
        return need > owned_[b] ? need - owned_[b] : 0;
    }
    void release(int b) {
        int* list = host_ + (size_t)b * max_pages_;
        for (int i = owned_[b] - 1; i >= 0; --i) free_.push_back(list[i]);
        owned_[b] = 0;
    }
    cudaError_t upload(cudaStream_t s) {
        const cudaError_t e = cudaMemcpyAsync(dev_, host_, (size_t)n_slots_ * max_pages_ * sizeof(int), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) dirty_ = false;
        return e;
    }
    bool dirty() const { return dirty_; }
    int n_pages() const { return n_pages_; }
    int page_rows() const { return page_rows_; }
    int max_pages() const { return max_pages_; }
    int free_count() const { return (int)free_.size(); }
    int owned(int b) const { return owned_[b]; }
    const int* list(int b) const { return host_ + (size_t)b * max_pages_; }
    int* host() const { return host_; }     // pinned [n_slots, max_pages] (+ the caller's extra ints behind it)
    int* device() const { return dev_; }    // device [n_slots, max_pages]

private:
    int n_pages_ = 0, page_rows_ = 0, n_slots_ = 0, max_pages_ = 0;
    int* dev_ = nullptr;
    int* host_ = nullptr;
    std::vector<int> free_, owned_;
    bool dirty_ = false;
};

}  // namespace b200
