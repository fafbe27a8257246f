// seq_cache.h — the paged per-position cache of the serving engine.  Every caching layer of the model gets one device
// array of n_pages * page_size rows; a sequence owns a list of pages (its page table, mirrored on the device) that
// grows as tokens arrive and goes back to the free list when the sequence ends.  Freed pages are handed out again
// first (a stack), so memory of finished requests is reused at once.
//
// Beside the rows a sequence may carry a block of fixed size (fp32 numbers: recurrent state, tails of convolutions, the
// previous token): one per slot, zeroed when the slot is opened, so a slot that is used again starts clean.  Models
// whose caching layers all look back a bounded number of positions let the engine trim: pages that lie wholly before
// the earliest position any later token can see go back to the free list while the sequence lives.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

class paged_cache {
  public:
    ~paged_cache();
    // dt: storage type of the rows; row_elems[i]: numbers per position of caching layer i
    // state_elems: fp32 numbers of per-sequence state (0: none)
    int init(int dt, const std::vector<int64_t> &row_elems, int64_t max_tokens, int page_size, int max_seqs, int64_t state_elems = 0);
    int open_seq();                         // slot (its state block zeroed), or -1 when all slots are taken
    int reserve(int slot, int64_t n_tokens); // pages for n_tokens positions (0 ok, -1: out of pages); table uploaded
    void close_seq(int slot);
    // gives back the pages that hold only positions < first_needed; their table entries stay but are never read again
    void trim(int slot, int64_t first_needed);
    float *state(int slot) const { return state_ ? state_ + (size_t)slot * (size_t)state_elems_ : nullptr; }
    int64_t state_elems() const { return state_elems_; }
    int live_pages(int slot) const;
    void *layer(int i) const { return layers_[(size_t)i]; }
    int n_layers() const { return (int)layers_.size(); }
    int page_size() const { return page_; }
    int64_t capacity_tokens() const { return (int64_t)n_pages_ * page_; }
    int free_pages() const { return (int)free_.size(); }
    int n_pages() const { return n_pages_; }
    const int32_t *table_dev(int slot) const { return tables_dev_ + (size_t)slot * (size_t)n_pages_; }
    const std::vector<int32_t> &table(int slot) const { return seqs_[(size_t)slot].pages; }
    const std::string &error() const { return err_; }

  private:
    struct seq {
        bool open = false;
        std::vector<int32_t> pages; // -1: trimmed
        size_t trimmed = 0;         // pages [0, trimmed) are given back
    };
    int dt_ = 0, page_ = 0, n_pages_ = 0;
    std::vector<void *> layers_;
    std::vector<int32_t> free_;
    std::vector<seq> seqs_;
    int32_t *tables_dev_ = nullptr;
    float *state_ = nullptr;
    int64_t state_elems_ = 0;
    std::string err_;
};
