// gemma_lm.cpp — the quantised Gemma model behind the serving engine's model interface (lm_model.h), registered as
// architecture "gemma": a folder whose config.json names a GGUF file ({"architecture": "gemma", "gguf": "model.gguf",
// "n_ctx": 2048}).  The Gemma path keeps its own position-major fp16 KV cache for ONE sequence (gemma_model.h), so it
// declares no rows in the paged cache and one live sequence; portions run through gemma_model::prefill (the dequant ->
// bf16 tcgen05 GEMMs), which computes the logits of every row.
#include <string>
#include <vector>

#include "gemma_model.h"
#include "lm_model.h"

namespace {

class gemma_lm : public lm_model {
  public:
    explicit gemma_lm(gemma_model *m) : m_(m) {}
    ~gemma_lm() override {
        if (rows_) ggb_buffer_free(rows_);
        if (out_) ggb_buffer_free(out_);
        delete m_;
    }
    const char *architecture() const override { return "gemma"; }
    int vocab() const override { return m_->config().n_vocab; }
    int dtype() const override { return GGB_TYPE_BF16; }
    std::vector<int64_t> cache_row_elems() const override { return {}; }
    int max_live_sequences() const override { return 1; }
    int bind_cache(paged_cache *, int64_t) override {
        int rc = m_->init_kv_cache();
        if (!rc) rc = m_->build_compute_graph(false, true);
        if (!rc) rc = ggb_buffer_alloc((size_t)max_portion() * 4, (void **)&rows_);
        if (!rc) rc = ggb_buffer_alloc((size_t)max_portion() * (size_t)vocab() * 4, (void **)&out_);
        if (rc) err_ = ggb_last_error();
        return rc;
    }
    int max_portion() const override { return 512; }
    int forward(const lm_portion &p, const int32_t *want, int n_want) override {
        if (p.pos0 + p.T > m_->config().n_ctx) {
            err_ = "the sequence leaves the model's context";
            return GGB_ERR_ARG;
        }
        int rc = m_->prefill(p.tokens, p.T, (int32_t)p.pos0, nullptr);
        if (!rc && n_want) rc = ggb_upload(rows_, want, (size_t)n_want * 4);
        if (!rc && n_want) rc = ggb_op_gather_rows_f32(m_->prefill_logits_dev(), rows_, n_want, vocab(), out_);
        if (rc) err_ = rc == GGB_ERR_UNSUPPORTED ? "this Gemma file (K-quants) has no batched prefill" : ggb_last_error();
        return rc;
    }
    const float *logits_dev() const override { return out_; }
    std::string last_error() const override { return err_; }

  private:
    gemma_model *m_;
    int32_t *rows_ = nullptr;
    float *out_ = nullptr;
    std::string err_;
};

lm_model *create_gemma(const std::string &dir, const json_value &cfg, const lm_load_options &, std::string *err) {
    const std::string file = cfg.string("gguf", "model.gguf");
    gemma_model *m = gemma_model::load_model_from_file((dir + "/" + file).c_str(), (int32_t)cfg.integer("n_ctx", 0), err);
    return m ? new gemma_lm(m) : nullptr;
}

struct register_gemma {
    register_gemma() { lm_register("gemma", &create_gemma); }
} g_register_gemma;

} // namespace
