// seq_cache.cpp — see seq_cache.h
#include "seq_cache.h"

#include <algorithm>

#include "ggml_b200.h"

paged_cache::~paged_cache() {
    for (void *p : layers_) ggb_buffer_free(p);
    if (tables_dev_) ggb_buffer_free(tables_dev_);
    if (state_) ggb_buffer_free(state_);
}

int paged_cache::init(int dt, const std::vector<int64_t> &row_elems, int64_t max_tokens, int page_size, int max_seqs, int64_t state_elems) {
    if (page_size <= 0 || max_tokens <= 0 || max_seqs <= 0 || !ggb_dtype_size(dt)) {
        err_ = "paged_cache: bad sizes";
        return GGB_ERR_ARG;
    }
    dt_ = dt;
    page_ = page_size;
    // a sequence may leave the end of its last page unused: one page of slack per slot
    n_pages_ = (int)((max_tokens + page_size - 1) / page_size) + max_seqs;
    seqs_.assign((size_t)max_seqs, seq());
    for (int p = n_pages_ - 1; p >= 0; p--) free_.push_back(p); // page 0 is handed out first
    for (int64_t e : row_elems) {
        void *d = nullptr;
        const size_t bytes = (size_t)n_pages_ * (size_t)page_ * (size_t)e * ggb_dtype_size(dt);
        int rc = ggb_buffer_alloc(bytes, &d);
        if (rc) {
            err_ = ggb_last_error();
            return rc;
        }
        layers_.push_back(d);
        if ((rc = ggb_buffer_memset(d, 0, bytes))) return rc;
    }
    int rc = ggb_buffer_alloc((size_t)max_seqs * (size_t)n_pages_ * 4, (void **)&tables_dev_);
    if (!rc && state_elems > 0) {
        state_elems_ = (state_elems + 3) / 4 * 4; // blocks stay 16-byte aligned
        rc = ggb_buffer_alloc((size_t)max_seqs * (size_t)state_elems_ * 4, (void **)&state_);
    }
    if (rc) err_ = ggb_last_error();
    return rc;
}

int paged_cache::open_seq() {
    for (size_t i = 0; i < seqs_.size(); i++)
        if (!seqs_[i].open) {
            seqs_[i].open = true;
            seqs_[i].pages.clear();
            seqs_[i].trimmed = 0;
            if (state_ && ggb_buffer_memset(state((int)i), 0, (size_t)state_elems_ * 4)) return -1; // stream-ordered: before the first step
            return (int)i;
        }
    return -1;
}

int paged_cache::reserve(int slot, int64_t n_tokens) {
    seq &s = seqs_[(size_t)slot];
    const size_t need = (size_t)((n_tokens + page_ - 1) / page_);
    const size_t had = s.pages.size();
    if (need <= had) return 0;
    if (need - had > free_.size()) {
        err_ = "paged_cache: out of pages (live sequences hold more tokens than the cache was sized for)";
        return -1;
    }
    if (need > (size_t)n_pages_) { // a page table holds n_pages entries: trimming frees pages, not positions
        err_ = "paged_cache: the sequence grows past the " + std::to_string((long long)n_pages_ * page_) + " positions the cache was sized for";
        return -1;
    }
    while (s.pages.size() < need) {
        s.pages.push_back(free_.back());
        free_.pop_back();
    }
    const int rc = ggb_upload(tables_dev_ + (size_t)slot * (size_t)n_pages_ + had, s.pages.data() + had, (need - had) * 4);
    if (rc) err_ = ggb_last_error();
    return rc;
}

void paged_cache::close_seq(int slot) {
    seq &s = seqs_[(size_t)slot];
    for (size_t i = s.pages.size(); i-- > 0;)
        if (s.pages[i] >= 0) free_.push_back(s.pages[i]); // the first page is reused first
    s.pages.clear();
    s.trimmed = 0;
    s.open = false;
}

void paged_cache::trim(int slot, int64_t first_needed) {
    seq &s = seqs_[(size_t)slot];
    if (first_needed <= 0) return;
    const size_t keep_from = std::min((size_t)(first_needed / page_), s.pages.size());
    for (size_t i = s.trimmed; i < keep_from; i++) {
        free_.push_back(s.pages[i]);
        s.pages[i] = -1;
    }
    if (keep_from > s.trimmed) s.trimmed = keep_from;
}

int paged_cache::live_pages(int slot) const {
    const seq &s = seqs_[(size_t)slot];
    return (int)(s.pages.size() - s.trimmed);
}
