// safolorn_model.h — the Safolorn decoder: parallel layers (x += mixer(norm1 x) + ff(norm2 x), both norms with a single
// number as weight), latent attention with a per-head sink and optional borrowing of another layer's cache, a clamped
// gated feed-forward or a mixture of experts, and a per-layer token side input.  Every size and constant comes from
// config.json or from a tensor's shape; the order of layers is the list in the configuration.
//
// The class lowers one portion of tokens to the ggb_op_* operators of the CUDA layer (dense.cu, latent_attention.cu,
// moe.cu), the same way gemma_model::prefill does for the quantised Gemma path; positions and page tables are read on
// the device, so the one-token step is captured into a CUDA graph and replayed.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "ggml_b200.h"
#include "lm_model.h"
#include "rotary.h"
#include "safetensors.h"

typedef rot_spec sf_rot; // rotary positions of a mixer (rotary.h)

struct sf_layer_cfg {
    // mixer
    int heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0;
    int kv_from = -1; // layer whose cache this layer reads, -1: its own
    float scale = 1.0f;
    sf_rot rot;
    // feed-forward: 0 none, 1 dense, 2 mixture of experts
    int mlp = 0;
    int ff = 0;
    float limit = 0.0f;
    int experts = 0, top = 0;
};

struct sf_config {
    int vocab = 0, width = 0, side_dim = 0;
    float eps = 1e-5f;
    std::vector<sf_layer_cfg> layers;
};
// fills *c from a parsed config.json; 0 or -1 with *err
int sf_parse_config(const json_value &j, sf_config *c, std::string *err);

struct sf_layer_w {
    float *norm1 = nullptr, *norm2 = nullptr; // fp32 (one number each, or a vector)
    int norm1_stride = 0, norm2_stride = 0;
    void *qd = nullptr;   // [H (D + Dr) (+ R + Dr)][W]: the query matrix with the layer's own down-projection stacked below
    float *dkv_norm = nullptr, *sink = nullptr;
    void *uk = nullptr, *uv = nullptr, *o = nullptr;
    void *gate_up = nullptr, *down = nullptr;            // dense: [2 ff][W], [W][ff]
    void *e_up = nullptr, *e_down = nullptr;             // experts stacked: [E][ff][W], [E][W][ff]
    float *router = nullptr, *router_b = nullptr;        // fp32
    void *side_gate = nullptr, *side_proj = nullptr;
    float *side_norm = nullptr;
    int cache_index = -1; // which array of the paged cache the layer reads (its own or the borrowed one)
    const float *cos_sin = nullptr;
};

class safolorn_model : public lm_model {
  public:
    static lm_model *create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err);
    // random weights of the configured sizes, generated on the host from `seed` (throughput runs; no file)
    static safolorn_model *create_random(const sf_config &cfg, const lm_load_options &opt, uint64_t seed, std::string *err);
    ~safolorn_model() override;

    const char *architecture() const override { return "Safolorn"; }
    int vocab() const override { return cfg_.vocab; }
    int dtype() const override { return dt_; }
    std::vector<int64_t> cache_row_elems() const override;
    int bind_cache(paged_cache *cache, int64_t max_positions) override;
    int max_portion() const override { return max_T_; }
    int forward(const lm_portion &p, const int32_t *want, int n_want) override;
    const float *logits_dev() const override { return logits_; }
    std::string last_error() const override { return err_; }

    const sf_config &config() const { return cfg_; }
    // keep the residual stream after every layer of the next forward calls (fp32 [layers][T][width] of the last portion)
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

  private:
    safolorn_model() {}
    int load(const safetensors_file *file, uint64_t seed);
    int alloc_scratch();
    int emit(int T, int n_split, const int32_t *table_dev, int n_want); // the operator sequence of one portion
    int upload_matrix(const std::vector<float> &host, void **dev);     // in dt_
    int upload_f32(const std::vector<float> &host, float **dev);
    int fail(int rc, const std::string &what);
    void free_all();

    sf_config cfg_;
    int dt_ = GGB_TYPE_BF16;
    int max_T_ = 1024;
    std::string err_;
    std::vector<sf_layer_w> lw_;
    void *embed_ = nullptr, *head_ = nullptr, *side_embed_ = nullptr;
    float *final_norm_ = nullptr;
    int final_norm_stride_ = 0;
    size_t weight_bytes_ = 0;
    std::vector<void *> owned_;
    paged_cache *cache_ = nullptr;
    int64_t max_pos_ = 0;
    std::map<std::string, float *> rot_tables_;
    // step inputs on the device
    int32_t *ids_ = nullptr, *pos0_ = nullptr, *want_ = nullptr, *table_cur_ = nullptr;
    // activations (sized for max_T_ tokens and the widest layer)
    float *x_ = nullptr, *qd_ = nullptr, *qa_ = nullptr, *part_ = nullptr, *attn_o_ = nullptr, *gu_ = nullptr, *ff_o_ = nullptr;
    void *h1_ = nullptr, *h2_ = nullptr, *ao_ = nullptr, *act_ = nullptr, *y1_ = nullptr, *hw_ = nullptr;
    float *y2_ = nullptr, *route_w_ = nullptr, *route_z_ = nullptr, *xw_ = nullptr, *logits_ = nullptr, *cap_ = nullptr;
    int32_t *route_i_ = nullptr, *group_ws_ = nullptr;
    int64_t part_rows_ = 0;
    bool capture_ = false;
    int cap_T_ = 0;
    int kernels_last_ = 0;
    // the one-token step as CUDA graphs: position and pages are read on the device, so one graph serves a sequence
    // until the number of splits of its visible positions changes (powers of two)
    struct step_graph {
        const int32_t *table;
        int n_split, n_want;
        ggb_graph *graph;
    };
    std::vector<step_graph> graphs_;
    bool use_graphs_ = true;
};
