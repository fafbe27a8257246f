// lm_engine.h — the serving loop around an lm_model: sequences by name, the paged cache that holds their state, the
// step function (every entry of a step brings the next tokens of one sequence; its portion is cut to what the model
// takes at once and run from the state earlier steps left), release of finished sequences, and greedy generation on
// top of the same step function.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "lm_model.h"
#include "seq_cache.h"

struct lm_entry {
    std::string id;
    std::vector<int32_t> tokens;
    std::vector<int32_t> want; // places among `tokens` whose logits are asked for, ascending or not
};

class lm_engine {
  public:
    // takes the model over; max_tokens: most tokens live sequences hold together; page_size / max_seqs: cache geometry
    int init(lm_model *model, int64_t max_tokens, int page_size, int max_seqs);
    // runs the entries one after the other; logits: rows in the order of the entries and of their `want` lists
    int step(const std::vector<lm_entry> &entries, const std::vector<std::string> &end, std::vector<float> *logits);
    // greedy continuation of a prompt through step(): first maximum of the last position's logits, n_new times
    int generate(const std::string &id, const std::vector<int32_t> &prompt, int n_new, std::vector<int32_t> *out);
    int64_t seq_len(const std::string &id) const;
    int seq_pages(const std::string &id, int32_t *out, int cap) const; // pages of a live sequence; returns how many
    int seq_live_pages(const std::string &id) const; // pages held now (after trimming); -1: no such sequence
    int live_seqs() const { return (int)seqs_.size(); }
    lm_model *model() const { return model_.get(); }
    paged_cache *cache() { return &cache_; }
    const std::string &error() const { return err_; }

  private:
    struct seq {
        int slot = -1;
        int64_t len = 0;
    };
    int run_entry(const lm_entry &e, std::vector<float> *logits, int32_t *greedy);
    std::unique_ptr<lm_model> model_;
    paged_cache cache_;
    std::map<std::string, seq> seqs_;
    int32_t *argmax_dev_ = nullptr;
    std::string err_;
};
