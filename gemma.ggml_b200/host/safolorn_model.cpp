// safolorn_model.cpp — see safolorn_model.h
#include "safolorn_model.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "lm_weights.h"
#include "seq_cache.h"

// an operator under the library's cudaEvent probes (ggb_prof_*), keyed by operator class like the Gemma path
#define SF_OP(name, expr)                              \
    do {                                               \
        ggb_prof_start(name);                          \
        const int rc__ = (expr);                       \
        ggb_prof_stop(name);                           \
        if (rc__ != 0) return fail(rc__, #expr);       \
    } while (0)

#define SF_TRY(expr)                                   \
    do {                                               \
        const int rc__ = (expr);                       \
        if (rc__ != 0) return fail(rc__, #expr);       \
    } while (0)

int safolorn_model::fail(int rc, const std::string &what) {
    if (err_.empty() || rc != GGB_ERR_ARG) err_ = what + ": " + ggb_last_error();
    return rc;
}

// ------------------------------------------------------------------------------------------------ configuration
int sf_parse_config(const json_value &j, sf_config *c, std::string *err) {
    auto bad = [&](const std::string &m) {
        if (err) *err = "config.json: " + m;
        return -1;
    };
    c->vocab = (int)j.integer("vocab", 0);
    c->width = (int)j.integer("width", 0);
    if (c->vocab <= 0 || c->width <= 0) return bad("vocab and width must be positive");
    if (const json_value *n = j.get("norm")) c->eps = (float)n->number("eps", 1e-5);
    if (const json_value *s = j.get("token_side")) c->side_dim = (int)s->integer("dim", 0);
    const json_value *layers = j.get("layers");
    if (!layers || layers->kind != json_value::ARR || layers->arr.empty()) return bad("'layers' must be a list");
    for (size_t i = 0; i < layers->arr.size(); i++) {
        const json_value &L = layers->arr[i];
        const std::string where = "layer " + std::to_string(i) + ": ";
        if (L.string("type", "") != "latent_attention") return bad(where + "unknown mixer type '" + L.string("type", "") + "'");
        const json_value *m = L.get("mixer");
        if (!m) return bad(where + "no 'mixer'");
        sf_layer_cfg l;
        l.heads = (int)m->integer("heads", 0);
        l.dim = (int)m->integer("dim", 0);
        l.rot_dim = (int)m->integer("rot_dim", 0);
        l.vdim = (int)m->integer("vdim", 0);
        l.kv_rank = (int)m->integer("kv_rank", 0);
        l.scale = (float)m->number("scale", 1.0);
        l.kv_from = m->get("kv_from") ? (int)m->integer("kv_from", -1) : -1;
        if (l.heads <= 0 || l.dim <= 0 || l.rot_dim < 0 || l.vdim <= 0 || l.kv_rank <= 0) return bad(where + "mixer sizes must be positive");
        if (const json_value *r = m->get("rot")) {
            l.rot.dims = (int)r->integer("dims", l.rot_dim);
            l.rot.base = r->number("base", 10000.0);
            if (const json_value *s = r->get("scaling")) {
                l.rot.scaled = true;
                l.rot.factor = s->number("factor", 1.0);
                l.rot.original = s->number("original", 0.0);
                l.rot.fast = s->number("fast", 32.0);
                l.rot.slow = s->number("slow", 1.0);
            }
        }
        if (l.rot.dims < 0 || l.rot.dims > l.rot_dim || l.rot.dims % 2) return bad(where + "rot.dims must be even and at most rot_dim");
        if (l.kv_from >= 0) {
            if (l.kv_from >= (int)i) return bad(where + "kv_from must name an earlier layer");
            const sf_layer_cfg &s = c->layers[(size_t)l.kv_from];
            if (s.kv_from >= 0 || s.kv_rank != l.kv_rank || s.rot_dim != l.rot_dim || s.rot.key() != l.rot.key())
                return bad(where + "kv_from must name a layer with its own cache and the same kv_rank, rot_dim and rotation");
        }
        if (const json_value *f = L.get("mlp")) {
            const std::string kind = f->string("kind", "");
            if (kind == "dense") {
                l.mlp = 1;
                l.ff = (int)f->integer("ff", 0);
                l.limit = f->get("limit") ? (float)f->number("limit", 0.0) : INFINITY; // no limit named: nothing is clamped
            } else if (kind == "moe") {
                l.mlp = 2;
                const json_value *e = f->get("expert"), *r = f->get("router");
                if (!e || !r) return bad(where + "a mixture of experts needs 'expert' and 'router'");
                l.ff = (int)e->integer("ff", 0);
                l.experts = (int)r->integer("experts", 0);
                l.top = (int)r->integer("top", 0);
                if (l.experts <= 0 || l.top <= 0 || l.top > l.experts) return bad(where + "need 0 < top <= experts");
            } else {
                return bad(where + "unknown mlp kind '" + kind + "'");
            }
            if (l.ff <= 0) return bad(where + "ff must be positive");
        }
        c->layers.push_back(l);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------ weights
int safolorn_model::upload_matrix(const std::vector<float> &host, void **dev) {
    const size_t n = host.size();
    void *d = nullptr;
    SF_TRY(ggb_buffer_alloc(std::max<size_t>(n, 1) * ggb_dtype_size(dt_), &d));
    owned_.push_back(d);
    if (dt_ == GGB_TYPE_BF16) {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = f32_to_bf16(host[i]);
        SF_TRY(ggb_upload(d, h.data(), n * 2));
        SF_TRY(ggb_sync());
    } else {
        SF_TRY(ggb_upload(d, host.data(), n * 4));
        SF_TRY(ggb_sync());
    }
    weight_bytes_ += n * ggb_dtype_size(dt_);
    *dev = d;
    return 0;
}

int safolorn_model::upload_f32(const std::vector<float> &host, float **dev) {
    void *d = nullptr;
    SF_TRY(ggb_buffer_alloc(std::max<size_t>(host.size(), 1) * 4, &d));
    owned_.push_back(d);
    SF_TRY(ggb_upload(d, host.data(), host.size() * 4));
    SF_TRY(ggb_sync());
    weight_bytes_ += host.size() * 4;
    *dev = (float *)d;
    return 0;
}

int safolorn_model::load(const safetensors_file *file, uint64_t seed) {
    const sf_config &c = cfg_;
    const int64_t W = c.width, V = c.vocab, L = (int64_t)c.layers.size();
    weight_source src{file, seed, &err_};
    std::vector<float> a, b;
#define SF_GET(...)                                 \
    do {                                            \
        if (src.get(__VA_ARGS__)) return GGB_ERR_ARG; \
    } while (0)
    auto norm_weight = [&](const std::string &name, float **dev, int *stride) -> int {
        const int n = src.numel(name, 1);
        if (n != 1 && n != W) {
            err_ = "tensor '" + name + "' must hold one number or one per coordinate";
            return GGB_ERR_ARG;
        }
        SF_GET(name, 1, n, 0.1f, 1.0f, &a);
        *stride = n == 1 ? 0 : 1;
        return upload_f32(a, dev);
    };
    const float aw = std::sqrt(3.0f / (float)W);
    SF_GET("embed", V, W, 1.7f, 0.f, &a);
    SF_TRY(upload_matrix(a, &embed_));
    SF_GET("head", V, W, aw, 0.f, &a);
    SF_TRY(upload_matrix(a, &head_));
    SF_TRY(norm_weight("final.norm", &final_norm_, &final_norm_stride_));
    if (c.side_dim > 0) {
        SF_GET("side.embed", V, L * c.side_dim, 1.7f, 0.f, &a);
        SF_TRY(upload_matrix(a, &side_embed_));
    }
    lw_.assign((size_t)L, sf_layer_w());
    int n_cache = 0;
    for (int64_t li = 0; li < L; li++) {
        const sf_layer_cfg &l = c.layers[(size_t)li];
        sf_layer_w &w = lw_[(size_t)li];
        const std::string p = "l" + std::to_string(li) + ".";
        const int64_t H = l.heads, D = l.dim, Dr = l.rot_dim, Dv = l.vdim, R = l.kv_rank, Nq = H * (D + Dr);
        SF_TRY(norm_weight(p + "norm1", &w.norm1, &w.norm1_stride));
        SF_GET(p + "mix.q", Nq, W, aw, 0.f, &a);
        if (l.kv_from < 0) {
            SF_GET(p + "mix.dkv", R + Dr, W, aw, 0.f, &b);
            a.insert(a.end(), b.begin(), b.end());
            SF_GET(p + "mix.dkv.norm", 1, R, 0.1f, 1.0f, &b);
            SF_TRY(upload_f32(b, &w.dkv_norm));
            w.cache_index = n_cache++;
        } else {
            w.cache_index = lw_[(size_t)l.kv_from].cache_index;
        }
        SF_TRY(upload_matrix(a, &w.qd));
        SF_GET(p + "mix.uk", H * D, R, std::sqrt(3.0f / (float)R), 0.f, &a);
        SF_TRY(upload_matrix(a, &w.uk));
        SF_GET(p + "mix.uv", H * Dv, R, std::sqrt(3.0f / (float)R), 0.f, &a);
        SF_TRY(upload_matrix(a, &w.uv));
        SF_GET(p + "mix.sink", 1, H, 1.0f, 0.f, &a);
        SF_TRY(upload_f32(a, &w.sink));
        SF_GET(p + "mix.o", W, H * Dv, std::sqrt(3.0f / (float)(H * Dv)), 0.f, &a);
        SF_TRY(upload_matrix(a, &w.o));
        if (l.mlp) SF_TRY(norm_weight(p + "norm2", &w.norm2, &w.norm2_stride));
        if (l.mlp == 1) {
            SF_GET(p + "mlp.gate", l.ff, W, aw, 0.f, &a);
            SF_GET(p + "mlp.up", l.ff, W, aw, 0.f, &b);
            a.insert(a.end(), b.begin(), b.end());
            SF_TRY(upload_matrix(a, &w.gate_up));
            SF_GET(p + "mlp.down", W, l.ff, std::sqrt(3.0f / (float)l.ff), 0.f, &a);
            SF_TRY(upload_matrix(a, &w.down));
        } else if (l.mlp == 2) {
            std::vector<float> up, down;
            for (int e = 0; e < l.experts; e++) {
                const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
                SF_GET(pe + "up", l.ff, W, aw, 0.f, &a);
                up.insert(up.end(), a.begin(), a.end());
                SF_GET(pe + "down", W, l.ff, std::sqrt(3.0f / (float)l.ff), 0.f, &a);
                down.insert(down.end(), a.begin(), a.end());
            }
            SF_TRY(upload_matrix(up, &w.e_up));
            SF_TRY(upload_matrix(down, &w.e_down));
            SF_GET(p + "mlp.router", l.experts, W, 2.0f * aw, 0.f, &a);
            SF_TRY(upload_f32(a, &w.router));
            if (!file || file->find(p + "mlp.router.b")) { // a router without a bias adds none
                SF_GET(p + "mlp.router.b", 1, l.experts, 0.5f, 0.f, &a);
                SF_TRY(upload_f32(a, &w.router_b));
            }
        }
        if (c.side_dim > 0) {
            SF_GET(p + "side.gate", c.side_dim, W, aw, 0.f, &a);
            SF_TRY(upload_matrix(a, &w.side_gate));
            SF_GET(p + "side.proj", W, c.side_dim, std::sqrt(3.0f / (float)c.side_dim), 0.f, &a);
            SF_TRY(upload_matrix(a, &w.side_proj));
            SF_GET(p + "side.norm", 1, W, 0.02f, 0.2f, &a);
            SF_TRY(upload_f32(a, &w.side_norm));
        }
    }
#undef SF_GET
    return 0;
}

lm_model *safolorn_model::create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err) {
    if (opt.random_weights) {
        sf_config c;
        std::string e;
        if (sf_parse_config(cfg, &c, &e)) {
            if (err) *err = e;
            return nullptr;
        }
        return create_random(c, opt, opt.seed, err);
    }
    safolorn_model *m = new safolorn_model();
    safetensors_file file;
    m->dt_ = opt.dtype;
    if (opt.max_portion > 0) m->max_T_ = opt.max_portion;
    int rc = sf_parse_config(cfg, &m->cfg_, &m->err_);
    if (!rc && !ggb_dtype_size(m->dt_)) rc = -1, m->err_ = "Safolorn runs in bfloat16 or float32";
    if (!rc) rc = file.open(dir + "/model.safetensors", &m->err_);
    if (!rc) rc = m->load(&file, 0);
    if (rc) {
        if (err) *err = m->err_;
        delete m;
        return nullptr;
    }
    return m;
}

safolorn_model *safolorn_model::create_random(const sf_config &cfg, const lm_load_options &opt, uint64_t seed, std::string *err) {
    safolorn_model *m = new safolorn_model();
    m->cfg_ = cfg;
    m->dt_ = opt.dtype;
    if (opt.max_portion > 0) m->max_T_ = opt.max_portion;
    if (!ggb_dtype_size(m->dt_) || m->load(nullptr, seed)) {
        if (err) *err = m->err_.empty() ? "Safolorn runs in bfloat16 or float32" : m->err_;
        delete m;
        return nullptr;
    }
    return m;
}

void safolorn_model::free_all() {
    for (step_graph &g : graphs_) ggb_graph_free(g.graph);
    graphs_.clear();
    for (void *p : owned_) ggb_buffer_free(p);
    owned_.clear();
}

safolorn_model::~safolorn_model() {
    ggb_sync();
    free_all();
}

std::vector<int64_t> safolorn_model::cache_row_elems() const {
    std::vector<int64_t> v;
    for (const sf_layer_cfg &l : cfg_.layers)
        if (l.kv_from < 0) v.push_back(ggb_latent_cache_ld(l.kv_rank, l.rot_dim));
    return v;
}

// ------------------------------------------------------------------------------------------------ buffers
int safolorn_model::alloc_scratch() {
    const sf_config &c = cfg_;
    const int64_t T = max_T_, W = c.width;
    int64_t nqd = 0, hqk = 0, hr = 0, hdv = 0, ff2 = 0, ffd = 0, slots = 0, effe = 0, ints = 0, top = 0, n_exp_max = 0;
    for (const sf_layer_cfg &l : c.layers) {
        const int64_t nq = (int64_t)l.heads * (l.dim + l.rot_dim) + (l.kv_from < 0 ? l.kv_rank + l.rot_dim : 0);
        nqd = std::max(nqd, nq);
        hqk = std::max(hqk, (int64_t)l.heads * (l.kv_rank + l.rot_dim));
        hr = std::max(hr, (int64_t)l.heads * (l.kv_rank + 2));
        hdv = std::max(hdv, (int64_t)l.heads * l.vdim);
        if (l.mlp == 1) ff2 = std::max(ff2, 2 * (int64_t)l.ff), ffd = std::max(ffd, (int64_t)l.ff);
        if (l.mlp == 2) {
            slots = std::max(slots, T * l.top);
            effe = std::max(effe, T * l.top * l.ff);
            ints = std::max(ints, (int64_t)ggb_moe_group_ints(T * l.top, l.experts));
            top = std::max(top, (int64_t)l.top);
            n_exp_max = std::max(n_exp_max, (int64_t)l.experts);
        }
    }
    part_rows_ = std::max<int64_t>(T, 320);
    const size_t es = ggb_dtype_size(dt_);
    auto alloc = [&](size_t bytes, void **p) -> int {
        SF_TRY(ggb_buffer_alloc(std::max<size_t>(bytes, 16), p));
        owned_.push_back(*p);
        return 0;
    };
#define SF_ALLOC(ptr, bytes) SF_TRY(alloc((size_t)(bytes), (void **)&(ptr)))
    SF_ALLOC(ids_, T * 4);
    SF_ALLOC(want_, T * 4);
    SF_ALLOC(pos0_, 16);
    SF_ALLOC(x_, T * W * 4);
    SF_ALLOC(h1_, T * W * es);
    SF_ALLOC(h2_, T * W * es);
    SF_ALLOC(qd_, T * nqd * 4);
    SF_ALLOC(qa_, T * hqk * 4);
    SF_ALLOC(part_, part_rows_ * hr * 4);
    SF_ALLOC(ao_, T * hdv * es);
    SF_ALLOC(attn_o_, T * W * 4);
    SF_ALLOC(ff_o_, T * W * 4);
    SF_ALLOC(gu_, T * ff2 * 4);
    SF_ALLOC(act_, T * ffd * es);
    SF_ALLOC(route_i_, T * top * 4);
    SF_ALLOC(route_w_, T * top * 4);
    SF_ALLOC(route_z_, T * n_exp_max * 4);
    SF_ALLOC(group_ws_, ints * 4);
    SF_ALLOC(y1_, effe * es);
    SF_ALLOC(y2_, slots * W * 4);
    SF_ALLOC(xw_, T * W * 4);
    SF_ALLOC(hw_, T * W * es);
    SF_ALLOC(logits_, T * (int64_t)c.vocab * 4);
#undef SF_ALLOC
    return 0;
}

int safolorn_model::bind_cache(paged_cache *cache, int64_t max_positions) {
    cache_ = cache;
    max_pos_ = max_positions;
    if ((int)cache_row_elems().size() != cache->n_layers()) return fail(GGB_ERR_ARG, "the cache has another number of layers than the model");
    for (size_t li = 0; li < cfg_.layers.size(); li++) {
        const sf_rot &r = cfg_.layers[li].rot;
        const std::string k = r.key();
        if (!rot_tables_.count(k)) {
            float *d = nullptr;
            const std::vector<float> t = rot_table(r, max_positions);
            SF_TRY(upload_f32(t.empty() ? std::vector<float>(1, 0.f) : t, &d));
            rot_tables_[k] = d;
        }
        lw_[li].cos_sin = rot_tables_[k];
    }
    return alloc_scratch();
}

// ------------------------------------------------------------------------------------------------ one portion
int safolorn_model::emit(int T, int ns, const int32_t *table, int n_want) {
    const sf_config &c = cfg_;
    const int64_t W = c.width, t = T;
    const int B = cache_->page_size();
    SF_OP("op_rows", ggb_op_embed_rows(dt_, embed_, ids_, t, W, x_));
    for (size_t li = 0; li < c.layers.size(); li++) {
        const sf_layer_cfg &l = c.layers[li];
        const sf_layer_w &w = lw_[li];
        const int H = l.heads, D = l.dim, Dr = l.rot_dim, Dv = l.vdim, R = l.kv_rank;
        const int64_t Nq = (int64_t)H * (D + Dr), Nqd = Nq + (l.kv_from < 0 ? R + Dr : 0);
        void *cache = cache_->layer(w.cache_index);
        // both branches norm the same x: one pass, two weights
        SF_OP("op_norm", ggb_op_rms_norm2(dt_, x_, W, w.norm1, w.norm1_stride, w.norm2, w.norm2_stride, c.eps, W, t, h1_, l.mlp ? h2_ : nullptr));
        SF_OP("op_linear", ggb_op_linear(dt_, w.qd, Nqd, W, h1_, W, t, qd_, Nqd));
        if (l.kv_from < 0)
            SF_OP("op_attn_prep", ggb_op_latent_kv_store(dt_, qd_ + Nq, Nqd, t, R, Dr, l.rot.dims, w.dkv_norm, c.eps, w.cos_sin, pos0_, table, B, cache));
        SF_OP("op_attn_prep", ggb_op_latent_q_absorb(dt_, qd_, Nqd, t, H, D, Dr, l.rot.dims, w.cos_sin, pos0_, w.uk, R, l.scale, qa_));
        SF_OP("op_attn", ggb_op_latent_attn(dt_, qa_, cache, table, B, pos0_, t, H, R, Dr, ns, part_));
        SF_OP("op_attn_out", ggb_op_latent_attn_out(dt_, part_, ns, w.sink, w.uv, t, H, R, Dv, ao_));
        SF_OP("op_linear", ggb_op_linear(dt_, w.o, W, (int64_t)H * Dv, ao_, (int64_t)H * Dv, t, attn_o_, W));
        if (l.mlp == 1) {
            SF_OP("op_linear", ggb_op_linear(dt_, w.gate_up, 2 * (int64_t)l.ff, W, h2_, W, t, gu_, 2 * (int64_t)l.ff));
            SF_OP("op_act", ggb_op_glu_clamp(dt_, gu_, l.ff, t, l.limit, 1.702f, act_));
            SF_OP("op_linear", ggb_op_linear(dt_, w.down, W, l.ff, act_, l.ff, t, ff_o_, W));
        } else if (l.mlp == 2) {
            SF_OP("op_moe", ggb_op_moe_route(dt_, h2_, W, t, w.router, w.router_b, l.experts, l.top, route_z_, route_i_, route_w_));
            SF_OP("op_moe", ggb_op_moe_group(route_i_, t, l.top, l.experts, group_ws_));
            SF_OP("op_moe_linear", ggb_op_moe_linear(dt_, w.e_up, l.ff, W, h2_, W, 1, t, l.top, l.experts, group_ws_, 1, y1_, l.ff));
            SF_OP("op_moe_linear", ggb_op_moe_linear(dt_, w.e_down, W, l.ff, y1_, l.ff, 0, t, l.top, l.experts, group_ws_, 0, y2_, W));
            SF_OP("op_moe", ggb_op_moe_combine(y2_, group_ws_, route_w_, t, l.top, l.experts, W, ff_o_));
        }
        SF_OP("op_residual", ggb_op_residual_side(dt_, x_, attn_o_, l.mlp ? ff_o_ : nullptr, W, t, ids_, side_embed_, (int64_t)c.layers.size() * c.side_dim,
                                    (int64_t)li * c.side_dim, c.side_dim, w.side_gate, w.side_proj, w.side_norm, c.eps));
        if (capture_ && cap_) SF_OP("op_rows", ggb_op_gather_rows_f32(x_, want_ + max_T_, t, W, cap_ + (size_t)li * (size_t)max_T_ * (size_t)W));
    }
    if (n_want > 0) {
        SF_OP("op_rows", ggb_op_gather_rows_f32(x_, want_, n_want, W, xw_));
        SF_OP("op_norm", ggb_op_rms_norm2(dt_, xw_, W, final_norm_, final_norm_stride_, nullptr, 0, c.eps, W, n_want, hw_, nullptr));
        SF_OP("op_linear", ggb_op_linear(dt_, head_, c.vocab, W, hw_, W, n_want, logits_, c.vocab));
    }
    return 0;
}

int safolorn_model::forward(const lm_portion &p, const int32_t *want, int n_want) {
    if (!cache_) return fail(GGB_ERR_ARG, "forward before bind_cache");
    if (p.T <= 0 || p.T > max_T_ || n_want < 0 || n_want > p.T || p.pos0 < 0 || p.pos0 + p.T > max_pos_) {
        err_ = "forward: a portion of " + std::to_string(p.T) + " tokens at position " + std::to_string(p.pos0) + " does not fit";
        return GGB_ERR_ARG;
    }
    for (int i = 0; i < p.T; i++)
        if (p.tokens[i] < 0 || p.tokens[i] >= cfg_.vocab) {
            err_ = "forward: token " + std::to_string(p.tokens[i]) + " is outside the vocabulary";
            return GGB_ERR_ARG;
        }
    const int32_t pos0 = (int32_t)p.pos0;
    SF_TRY(ggb_upload(ids_, p.tokens, (size_t)p.T * 4));
    SF_TRY(ggb_upload(pos0_, &pos0, 4));
    if (n_want) SF_TRY(ggb_upload(want_, want, (size_t)n_want * 4));
    // splits of the visible positions: enough CTAs for a short portion, one split once the tokens fill the GPU
    const int64_t n_kv = p.pos0 + p.T;
    int64_t ns = std::min<int64_t>((n_kv + (p.T <= 8 ? 31 : 127)) / (p.T <= 8 ? 32 : 128), std::max<int64_t>(1, 296 / p.T));
    ns = std::max<int64_t>(1, std::min<int64_t>(ns, 64));
    if (p.T == 1) { // powers of two: the captured one-token step changes rarely
        int64_t q = 1;
        while (q < ns) q *= 2;
        ns = q;
    }
    while (ns > 1 && ns * p.T > part_rows_) ns--;
    const int64_t l0 = ggb_launch_count();
    if (capture_) {
        if (!cap_) {
            void *d = nullptr;
            SF_TRY(ggb_buffer_alloc(cfg_.layers.size() * (size_t)max_T_ * (size_t)cfg_.width * 4, &d));
            owned_.push_back(d);
            cap_ = (float *)d;
            // identity row list behind the wanted rows: the capture copies whole portions with the gather operator
            std::vector<int32_t> iota((size_t)max_T_);
            for (int i = 0; i < max_T_; i++) iota[(size_t)i] = i;
            void *w2 = nullptr;
            SF_TRY(ggb_buffer_alloc((size_t)max_T_ * 8, &w2));
            owned_.push_back(w2);
            want_ = (int32_t *)w2;
            SF_TRY(ggb_upload(want_ + max_T_, iota.data(), (size_t)max_T_ * 4));
            if (n_want) SF_TRY(ggb_upload(want_, want, (size_t)n_want * 4));
        }
        cap_T_ = p.T;
    }
    if (p.T == 1 && use_graphs_ && !capture_ && !getenv("GGB_SF_NO_GRAPH")) {
        ggb_graph *g = nullptr;
        for (const step_graph &sg : graphs_)
            if (sg.table == p.block_table_dev && sg.n_split == (int)ns && sg.n_want == n_want) g = sg.graph;
        if (!g) {
            SF_TRY(ggb_capture_begin());
            const int rc = emit(1, (int)ns, p.block_table_dev, n_want);
            const int rc2 = ggb_capture_end(&g);
            if (rc) return rc;
            if (rc2) return fail(rc2, "ggb_capture_end");
            if (graphs_.size() >= 32) {
                ggb_graph_free(graphs_.front().graph);
                graphs_.erase(graphs_.begin());
            }
            graphs_.push_back(step_graph{p.block_table_dev, (int)ns, n_want, g});
        }
        SF_TRY(ggb_graph_launch(g));
    } else {
        SF_TRY(emit(p.T, (int)ns, p.block_table_dev, n_want));
    }
    kernels_last_ = (int)(ggb_launch_count() - l0);
    return 0;
}

int safolorn_model::get_capture(int layer, float *host, int64_t n) const {
    if (!cap_ || layer < 0 || layer >= (int)cfg_.layers.size() || n > (int64_t)cap_T_ * cfg_.width) return GGB_ERR_ARG;
    return ggb_download(host, cap_ + (size_t)layer * (size_t)max_T_ * (size_t)cfg_.width, (size_t)n * 4);
}

namespace {
struct register_safolorn {
    register_safolorn() { lm_register("Safolorn", &safolorn_model::create); }
} g_register_safolorn;
} // namespace
