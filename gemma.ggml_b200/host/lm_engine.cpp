// lm_engine.cpp — see lm_engine.h
#include "lm_engine.h"

#include <algorithm>

#include "ggml_b200.h"

int lm_engine::init(lm_model *model, int64_t max_tokens, int page_size, int max_seqs) {
    model_.reset(model);
    if (model->max_live_sequences() > 0) max_seqs = std::min(max_seqs, model->max_live_sequences());
    int rc = cache_.init(model->dtype(), model->cache_row_elems(), max_tokens, page_size, max_seqs, model->state_elems());
    if (rc) {
        err_ = cache_.error();
        return rc;
    }
    if ((rc = model->bind_cache(&cache_, cache_.capacity_tokens()))) {
        err_ = model->last_error();
        return rc;
    }
    if ((rc = ggb_buffer_alloc(16, (void **)&argmax_dev_))) err_ = ggb_last_error();
    return rc;
}

int64_t lm_engine::seq_len(const std::string &id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? -1 : it->second.len;
}

int lm_engine::seq_pages(const std::string &id, int32_t *out, int cap) const {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return -1;
    const std::vector<int32_t> &t = cache_.table(it->second.slot);
    for (int i = 0; i < cap && i < (int)t.size(); i++) out[i] = t[(size_t)i];
    return (int)t.size();
}

int lm_engine::run_entry(const lm_entry &e, std::vector<float> *logits, int32_t *greedy) {
    auto it = seqs_.find(e.id);
    if (it == seqs_.end()) {
        seq s;
        s.slot = cache_.open_seq();
        if (s.slot < 0) {
            err_ = "no free sequence slot for '" + e.id + "' (or its state could not be cleared)";
            return GGB_ERR_ARG;
        }
        it = seqs_.emplace(e.id, s).first;
    }
    seq &s = it->second;
    const int64_t n = (int64_t)e.tokens.size();
    for (int32_t w : e.want)
        if (w < 0 || w >= n) {
            err_ = "entry '" + e.id + "': a wanted place is outside its tokens";
            return GGB_ERR_ARG;
        }
    if (cache_.reserve(s.slot, s.len + n)) {
        err_ = cache_.error();
        return GGB_ERR_ARG;
    }
    const int V = model_->vocab(), step = model_->max_portion();
    const size_t out0 = logits ? logits->size() : 0;
    if (logits) logits->resize(out0 + e.want.size() * (size_t)V);
    // cut the portion into what the model takes at once; every cut answers the wanted places that fall into it
    for (int64_t lo = 0; lo < n; lo += step) {
        const int64_t hi = std::min(n, lo + step);
        std::vector<int32_t> rows, slots;
        for (size_t k = 0; k < e.want.size(); k++)
            if (e.want[k] >= lo && e.want[k] < hi) {
                rows.push_back((int32_t)(e.want[k] - lo));
                slots.push_back((int32_t)k);
            }
        lm_portion p;
        p.tokens = e.tokens.data() + lo;
        p.T = (int)(hi - lo);
        p.pos0 = s.len + lo;
        p.block_table_dev = cache_.table_dev(s.slot);
        p.state_dev = cache_.state(s.slot);
        int rc = model_->forward(p, rows.data(), (int)rows.size());
        if (rc) {
            err_ = model_->last_error();
            return rc;
        }
        if (logits && !rows.empty()) {
            std::vector<float> tmp(rows.size() * (size_t)V);
            if ((rc = ggb_download(tmp.data(), model_->logits_dev(), tmp.size() * 4))) {
                err_ = ggb_last_error();
                return rc;
            }
            for (size_t r = 0; r < rows.size(); r++)
                std::copy(tmp.begin() + (ptrdiff_t)(r * (size_t)V), tmp.begin() + (ptrdiff_t)((r + 1) * (size_t)V),
                          logits->begin() + (ptrdiff_t)(out0 + (size_t)slots[r] * (size_t)V));
        }
        if (greedy && hi == n && !rows.empty()) { // the sampler: first maximum of the last wanted row, on the device
            if ((rc = ggb_op_argmax(model_->logits_dev() + (rows.size() - 1) * (size_t)V, V, argmax_dev_)) ||
                (rc = ggb_download(greedy, argmax_dev_, 4))) {
                err_ = ggb_last_error();
                return rc;
            }
        }
    }
    s.len += n;
    // rows no later token can see: their pages serve other sequences from now on
    if (model_->cache_lookback() > 0) cache_.trim(s.slot, s.len - model_->cache_lookback() + 1);
    return 0;
}

int lm_engine::seq_live_pages(const std::string &id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? -1 : cache_.live_pages(it->second.slot);
}

int lm_engine::step(const std::vector<lm_entry> &entries, const std::vector<std::string> &end, std::vector<float> *logits) {
    if (logits) logits->clear();
    for (const lm_entry &e : entries) {
        if (e.tokens.empty()) continue;
        const int rc = run_entry(e, logits, nullptr);
        if (rc) return rc;
    }
    for (const std::string &id : end) {
        auto it = seqs_.find(id);
        if (it == seqs_.end()) continue;
        cache_.close_seq(it->second.slot);
        seqs_.erase(it);
    }
    return ggb_sync();
}

int lm_engine::generate(const std::string &id, const std::vector<int32_t> &prompt, int n_new, std::vector<int32_t> *out) {
    out->clear();
    if (prompt.empty()) {
        err_ = "generate: empty prompt";
        return GGB_ERR_ARG;
    }
    lm_entry e;
    e.id = id;
    e.tokens = prompt;
    e.want.push_back((int32_t)prompt.size() - 1);
    for (int i = 0; i < n_new; i++) {
        int32_t next = -1;
        const int rc = run_entry(e, nullptr, &next);
        if (rc) return rc;
        out->push_back(next);
        e.tokens.assign(1, next);
        e.want.assign(1, 0);
    }
    return 0;
}
