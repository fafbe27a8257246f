// begupel_model.h — the Begupel decoder: a hashed bigram row added to the token embedding; layers that norm the
// sublayer's OUTPUT (x += norm1(mixer(x)), x += norm2(ff(x)), both RMS norms in groups); a causal convolution over time
// in front of every mixer; two kinds of mixer in any order: "lightning" (linear attention with a fixed decay per
// head, gated) and "parallel" (sliding-window soft-max attention with rotated values beside a gated delta rule, summed
// with two scales); an optional dense ReLU-gated feed-forward with biases; soft-capped logits.  Every size and
// constant comes from config.json or a tensor's shape.
//
// What a sequence carries: rows [k | rotated v] of the window attentions in the engine's paged cache (pages behind every
// window go back to the pool while the sequence lives), and one block of fp32 state in the cache's per-sequence
// storage: the previous token, the convolutions' tails and the matrices S of both recurrences.
//
// The class lowers a portion of tokens to ggb_op_* operators (dense.cu, recurrent.cu, window_attention.cu), as
// safolorn_model does; positions, page tables and state are read on the device, so the one-token step is captured
// into a CUDA graph per sequence slot and replayed.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "ggml_b200.h"
#include "lm_model.h"
#include "rotary.h"
#include "safetensors.h"

struct bg_window_cfg { // soft-max attention over a sliding window
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    int64_t window = 0; // 0: every earlier position
    float scale = 1.0f;
    rot_spec rot;       // of q and k; rot.dims == 0: none
    rot_spec vrot;      // of the values: all vdim coordinates, the same base, never rescaled; dims == 0: none
};

struct bg_delta_cfg { // gated delta rule
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0, conv = 1;
};

struct bg_layer_cfg {
    int type = 0; // 0 lightning, 1 parallel
    int heads = 0, dim = 0, vdim = 0; // lightning
    std::vector<float> decay;
    bg_window_cfg left;
    bg_delta_cfg right;
    float left_scale = 1.0f, right_scale = 1.0f;
    int ff = 0; // 0: the layer has no feed-forward
};

struct bg_config {
    int vocab = 0, width = 0, groups = 1, taps = 0;
    float eps = 1e-5f, softcap = 0.0f; // softcap 0: logits as they are
    int64_t buckets = 0, mul_prev = 0, mul_cur = 0; // buckets 0: no bigram table
    std::vector<bg_layer_cfg> layers;
};
int bg_parse_config(const json_value &j, bg_config *c, std::string *err);

struct bg_layer_w {
    float *canon = nullptr, *norm1 = nullptr, *norm2 = nullptr;
    void *proj = nullptr; // every matrix that reads the mixer's input, stacked (rows padded to a multiple of 32)
    int64_t n_proj = 0;
    // column offsets into a row of the stacked product
    int64_t o_q = 0, o_k = 0, o_v = 0, o_g = 0, o_rq = 0, o_rk = 0, o_rv = 0, o_rg = 0, o_rb = 0, o_ra = 0;
    float *decay = nullptr, *mix_norm = nullptr;                      // lightning
    void *o = nullptr;                                                // lightning / left output projection
    float *qn = nullptr, *kn = nullptr;                               // left
    const float *cs_k = nullptr, *cs_v = nullptr;
    int cache_index = -1;
    float *rconv = nullptr, *A_log = nullptr, *dt_bias = nullptr, *rnorm = nullptr; // right
    void *ro = nullptr;
    void *gate_up = nullptr, *down = nullptr;                         // feed-forward
    float *gate_b = nullptr, *up_b = nullptr, *down_b = nullptr;
    // offsets (fp32 numbers) into the sequence's state block
    int64_t s_canon = 0, s_rconv = 0, s_S = 0;
};

class begupel_model : public lm_model {
  public:
    static lm_model *create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err);
    ~begupel_model() override;

    const char *architecture() const override { return "Begupel"; }
    int vocab() const override { return cfg_.vocab; }
    int dtype() const override { return dt_; }
    std::vector<int64_t> cache_row_elems() const override;
    int64_t state_elems() const override { return state_elems_; }
    int64_t cache_lookback() const override { return lookback_; }
    int bind_cache(paged_cache *cache, int64_t max_positions) override;
    int max_portion() const override { return max_T_; }
    int forward(const lm_portion &p, const int32_t *want, int n_want) override;
    const float *logits_dev() const override { return logits_; }
    std::string last_error() const override { return err_; }
    int set_capture(bool on) override {
        capture_ = on;
        return 0;
    }
    int set_use_graphs(bool on) override {
        use_graphs_ = on;
        return 0;
    }
    int get_capture(int layer, float *host, int64_t n) const override;
    size_t weight_bytes() const override { return weight_bytes_; }
    int kernels_last_forward() const override { return kernels_last_; }
    const bg_config &config() const { return cfg_; }

  private:
    begupel_model() {}
    int load(const safetensors_file *file, uint64_t seed);
    int alloc_scratch();
    int emit(int T, const int32_t *table_dev, float *state, int n_want);
    int upload_matrix(const std::vector<float> &host, void **dev);
    int upload_f32(const std::vector<float> &host, float **dev);
    int fail(int rc, const std::string &what);

    bg_config cfg_;
    int dt_ = GGB_TYPE_BF16;
    int max_T_ = 1024;
    std::string err_;
    std::vector<bg_layer_w> lw_;
    void *embed_ = nullptr, *bigram_ = nullptr, *head_ = nullptr;
    float *final_norm_ = nullptr;
    size_t weight_bytes_ = 0;
    int64_t state_elems_ = 0, lookback_ = 0;
    std::vector<void *> owned_;
    paged_cache *cache_ = nullptr;
    int64_t max_pos_ = 0;
    std::map<std::string, float *> rot_tables_;
    int32_t *ids_ = nullptr, *pos0_ = nullptr, *want_ = nullptr, *iota_ = nullptr;
    float *x_ = nullptr, *pr_ = nullptr, *cv_ = nullptr, *qr_ = nullptr, *ro_ = nullptr, *ya_ = nullptr, *yb_ = nullptr, *gu_ = nullptr,
          *xw_ = nullptr, *logits_ = nullptr, *cap_ = nullptr, *wa_ = nullptr;
    void *h_ = nullptr, *ao_ = nullptr, *gd_ = nullptr, *xd_ = nullptr, *act_ = nullptr, *hw_ = nullptr;
    bool capture_ = false, use_graphs_ = true;
    int cap_T_ = 0, kernels_last_ = 0;
    struct step_graph {
        const int32_t *table;
        const float *state;
        int n_want;
        ggb_graph *graph;
    };
    std::vector<step_graph> graphs_;
};
