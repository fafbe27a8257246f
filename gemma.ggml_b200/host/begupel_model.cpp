// begupel_model.cpp — see begupel_model.h
#include "begupel_model.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "lm_weights.h"
#include "seq_cache.h"

#define BG_OP(name, expr)                        \
    do {                                         \
        ggb_prof_start(name);                    \
        const int rc__ = (expr);                 \
        ggb_prof_stop(name);                     \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

#define BG_TRY(expr)                             \
    do {                                         \
        const int rc__ = (expr);                 \
        if (rc__ != 0) return fail(rc__, #expr); \
    } while (0)

int begupel_model::fail(int rc, const std::string &what) {
    if (err_.empty() || rc != GGB_ERR_ARG) err_ = what + ": " + ggb_last_error();
    return rc;
}

// ------------------------------------------------------------------------------------------------ configuration
int bg_parse_config(const json_value &j, bg_config *c, std::string *err) {
    auto bad = [&](const std::string &m) {
        if (err) *err = "config.json: " + m;
        return -1;
    };
    c->vocab = (int)j.integer("vocab", 0);
    c->width = (int)j.integer("width", 0);
    if (c->vocab <= 0 || c->width <= 0) return bad("vocab and width must be positive");
    if (const json_value *n = j.get("norm")) {
        c->eps = (float)n->number("eps", 1e-5);
        c->groups = (int)n->integer("groups", 1);
    }
    if (c->groups <= 0 || c->width % c->groups) return bad("norm.groups must divide the width");
    if (const json_value *k = j.get("canon")) c->taps = (int)k->integer("taps", 0);
    if (c->taps < 0 || c->taps > 8) return bad("canon.taps must be between 0 and 8");
    if (const json_value *e = j.get("embedding"))
        if (const json_value *b = e->get("bigram")) {
            c->buckets = b->integer("buckets", 0);
            c->mul_prev = b->integer("mul_prev", 0);
            c->mul_cur = b->integer("mul_cur", 0);
            if (c->buckets <= 0) return bad("embedding.bigram.buckets must be positive");
        }
    c->softcap = (float)j.number("logit_softcap", 0.0);
    if (c->softcap < 0.f) return bad("logit_softcap must be positive");
    const json_value *layers = j.get("layers");
    if (!layers || layers->kind != json_value::ARR || layers->arr.empty()) return bad("'layers' must be a list");
    for (size_t i = 0; i < layers->arr.size(); i++) {
        const json_value &L = layers->arr[i];
        const std::string where = "layer " + std::to_string(i) + ": ";
        const std::string type = L.string("type", "");
        const json_value *m = L.get("mixer");
        if (!m) return bad(where + "no 'mixer'");
        bg_layer_cfg l;
        if (type == "lightning") {
            l.type = 0;
            l.heads = (int)m->integer("heads", 0);
            l.dim = (int)m->integer("dim", 0);
            l.vdim = (int)m->integer("vdim", 0);
            if (l.heads <= 0 || l.dim <= 0 || l.vdim <= 0) return bad(where + "mixer sizes must be positive");
            const json_value *d = m->get("decay");
            if (d && d->kind == json_value::NUM) { // one number: every head forgets at the same rate
                l.decay.assign((size_t)l.heads, (float)d->num);
            } else {
                if (!d || d->kind != json_value::ARR || (int)d->arr.size() != l.heads) return bad(where + "'decay' must list one number per head");
                for (const json_value &v : d->arr) {
                    if (v.kind != json_value::NUM) return bad(where + "'decay' must list numbers");
                    l.decay.push_back((float)v.num);
                }
            }
        } else if (type == "parallel") {
            l.type = 1;
            const json_value *a = m->get("left"), *r = m->get("right");
            if (!a || !r) return bad(where + "a parallel mixer needs 'left' and 'right'");
            l.left_scale = (float)m->number("left_scale", 1.0);
            l.right_scale = (float)m->number("right_scale", 1.0);
            bg_window_cfg &w = l.left;
            w.heads = (int)a->integer("heads", 0);
            w.kv_heads = (int)a->integer("kv_heads", w.heads);
            w.dim = (int)a->integer("dim", 0);
            w.vdim = (int)a->integer("vdim", w.dim);
            w.scale = (float)a->number("scale", 1.0);
            if (const json_value *k = a->get("mask")) w.window = k->integer("size", 0);
            if (w.heads <= 0 || w.kv_heads <= 0 || w.heads % w.kv_heads || w.dim <= 0 || w.vdim <= 0 || w.window < 0)
                return bad(where + "left: sizes must be positive and kv_heads must divide heads");
            if (w.dim % 2 || w.vdim % 2) return bad(where + "left: dim and vdim must be even");
            if (const json_value *ro = a->get("rot")) {
                w.rot.dims = (int)ro->integer("dims", w.dim);
                w.rot.base = ro->number("base", 10000.0);
                if (const json_value *s = ro->get("scaling")) {
                    w.rot.linear = true;
                    w.rot.factor = s->number("factor", 1.0);
                    if (!(w.rot.factor > 0.0)) return bad(where + "left: rot.scaling.factor must be positive");
                }
                if (w.rot.dims < 0 || w.rot.dims > w.dim || w.rot.dims % 2) return bad(where + "left: rot.dims must be even and at most dim");
                w.vrot.dims = w.vdim;
                w.vrot.base = w.rot.base;
            }
            bg_delta_cfg &d = l.right;
            d.heads = (int)r->integer("heads", 0);
            d.kv_heads = (int)r->integer("kv_heads", d.heads);
            d.dim = (int)r->integer("dim", 0);
            d.vdim = (int)r->integer("vdim", d.dim);
            d.conv = (int)r->integer("conv", 1);
            if (d.heads <= 0 || d.kv_heads <= 0 || d.heads % d.kv_heads || d.dim <= 0 || d.vdim <= 0)
                return bad(where + "right: sizes must be positive and kv_heads must divide heads");
            if (d.conv < 1 || d.conv > 8) return bad(where + "right: conv must be between 1 and 8 taps");
            if (d.dim > 256) return bad(where + "right: dim above 256 is not built");
        } else {
            return bad(where + "unknown mixer type '" + type + "'");
        }
        if (l.type == 0 && l.dim > 256) return bad(where + "dim above 256 is not built");
        if (const json_value *f = L.get("mlp")) {
            const std::string kind = f->string("kind", "");
            if (kind != "dense") return bad(where + "unknown mlp kind '" + kind + "'");
            l.ff = (int)f->integer("ff", 0);
            if (l.ff <= 0) return bad(where + "ff must be positive");
        }
        c->layers.push_back(l);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------ weights
int begupel_model::upload_matrix(const std::vector<float> &host, void **dev) {
    const size_t n = host.size();
    void *d = nullptr;
    BG_TRY(ggb_buffer_alloc(std::max<size_t>(n, 8) * ggb_dtype_size(dt_), &d));
    owned_.push_back(d);
    if (dt_ == GGB_TYPE_BF16) {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = f32_to_bf16(host[i]);
        BG_TRY(ggb_upload(d, h.data(), n * 2));
        BG_TRY(ggb_sync());
    } else {
        BG_TRY(ggb_upload(d, host.data(), n * 4));
        BG_TRY(ggb_sync());
    }
    weight_bytes_ += n * ggb_dtype_size(dt_);
    *dev = d;
    return 0;
}

int begupel_model::upload_f32(const std::vector<float> &host, float **dev) {
    void *d = nullptr;
    BG_TRY(ggb_buffer_alloc(std::max<size_t>(host.size(), 4) * 4, &d));
    owned_.push_back(d);
    BG_TRY(ggb_upload(d, host.data(), host.size() * 4));
    BG_TRY(ggb_sync());
    weight_bytes_ += host.size() * 4;
    *dev = (float *)d;
    return 0;
}

int begupel_model::load(const safetensors_file *file, uint64_t seed) {
    const bg_config &c = cfg_;
    const int64_t W = c.width, V = c.vocab;
    weight_source src{file, seed, &err_};
    std::vector<float> a, b;
#define BG_GET(...)                                   \
    do {                                              \
        if (src.get(__VA_ARGS__)) return GGB_ERR_ARG; \
    } while (0)
#define BG_F32(name, n, amp, mean, dst)  \
    do {                                 \
        BG_GET(name, 1, n, amp, mean, &a); \
        BG_TRY(upload_f32(a, dst));      \
    } while (0)
    const float aw = std::sqrt(3.0f / (float)W);
    auto amp = [](int64_t fan_in) { return std::sqrt(3.0f / (float)fan_in); };
    BG_GET("embed", V, W, 1.7f, 0.f, &a);
    BG_TRY(upload_matrix(a, &embed_));
    if (c.buckets > 0) {
        BG_GET("bigram", c.buckets + 1, W, 1.0f, 0.f, &a);
        BG_TRY(upload_matrix(a, &bigram_));
    }
    BG_GET("head", V, W, aw, 0.f, &a);
    BG_TRY(upload_matrix(a, &head_));
    BG_F32("final.norm", W, 0.1f, 1.0f, &final_norm_);
    lw_.assign(c.layers.size(), bg_layer_w());
    int n_cache = 0;
    int64_t st = 4; // number 0 of the block: the previous token
    auto take = [&](int64_t n) {
        const int64_t at = st;
        st += (n + 3) / 4 * 4;
        return at;
    };
    // stacks `name` (rows x W) below what `stack` already holds; returns the row it starts at
    std::vector<float> stack;
    auto push = [&](const std::string &name, int64_t rows, float amplitude, int64_t *at) -> int {
        *at = (int64_t)(stack.size() / (size_t)W);
        if (src.get(name, rows, W, amplitude, 0.f, &b)) return GGB_ERR_ARG;
        stack.insert(stack.end(), b.begin(), b.end());
        return 0;
    };
    for (size_t li = 0; li < c.layers.size(); li++) {
        const bg_layer_cfg &l = c.layers[li];
        bg_layer_w &w = lw_[li];
        const std::string p = "l" + std::to_string(li) + ".";
        BG_F32(p + "norm1", W, 0.1f, 1.0f, &w.norm1);
        if (c.taps > 0) {
            BG_F32(p + "canon1", W * c.taps, 0.3f, 0.f, &w.canon);
            w.s_canon = take((int64_t)(c.taps - 1) * W);
        } else { // no convolution: one tap of weight zero leaves h = x
            BG_TRY(upload_f32(std::vector<float>((size_t)W, 0.f), &w.canon));
        }
        stack.clear();
        if (l.type == 0) {
            const int64_t H = l.heads, D = l.dim, Dv = l.vdim;
            BG_TRY(push(p + "mix.q", H * D, aw, &w.o_q));
            BG_TRY(push(p + "mix.k", H * D, aw, &w.o_k));
            BG_TRY(push(p + "mix.v", H * Dv, aw, &w.o_v));
            BG_TRY(push(p + "mix.g", H * Dv, aw, &w.o_g));
            BG_F32(p + "mix.norm", H * Dv, 0.1f, 1.0f, &w.mix_norm);
            BG_GET(p + "mix.o", W, H * Dv, amp(H * Dv), 0.f, &a);
            BG_TRY(upload_matrix(a, &w.o));
            BG_TRY(upload_f32(l.decay, &w.decay));
            w.s_S = take(H * D * Dv);
        } else {
            const bg_window_cfg &A = l.left;
            const bg_delta_cfg &R = l.right;
            const int64_t H = A.heads, G = A.kv_heads, D = A.dim, Dv = A.vdim;
            const int64_t Hr = R.heads, Gr = R.kv_heads, Dr = R.dim, Dvr = R.vdim, C = 2 * Gr * Dr + Hr * Dvr;
            BG_TRY(push(p + "mix.left.q", H * D, aw, &w.o_q));
            BG_TRY(push(p + "mix.left.k", G * D, aw, &w.o_k));
            BG_TRY(push(p + "mix.left.v", G * Dv, aw, &w.o_v));
            BG_TRY(push(p + "mix.right.q", Gr * Dr, aw, &w.o_rq));
            BG_TRY(push(p + "mix.right.k", Gr * Dr, aw, &w.o_rk));
            BG_TRY(push(p + "mix.right.v", Hr * Dvr, aw, &w.o_rv));
            BG_TRY(push(p + "mix.right.g", Hr * Dvr, aw, &w.o_rg));
            BG_TRY(push(p + "mix.right.b", Hr, aw, &w.o_rb));
            BG_TRY(push(p + "mix.right.a", Hr, aw, &w.o_ra));
            BG_F32(p + "mix.left.q.norm", H * D, 0.1f, 1.0f, &w.qn);
            BG_F32(p + "mix.left.k.norm", G * D, 0.1f, 1.0f, &w.kn);
            BG_GET(p + "mix.left.o", W, H * Dv, amp(H * Dv), 0.f, &a);
            BG_TRY(upload_matrix(a, &w.o));
            w.cache_index = n_cache++;
            // the three convolutions side by side, as their channels lie in the stacked product
            std::vector<float> cw;
            BG_GET(p + "mix.right.q.conv", Gr * Dr, R.conv, 0.5f, 0.f, &a);
            cw.insert(cw.end(), a.begin(), a.end());
            BG_GET(p + "mix.right.k.conv", Gr * Dr, R.conv, 0.5f, 0.f, &a);
            cw.insert(cw.end(), a.begin(), a.end());
            BG_GET(p + "mix.right.v.conv", Hr * Dvr, R.conv, 0.5f, 0.f, &a);
            cw.insert(cw.end(), a.begin(), a.end());
            BG_TRY(upload_f32(cw, &w.rconv));
            BG_F32(p + "mix.right.A_log", Hr, 1.0f, -1.0f, &w.A_log);
            BG_F32(p + "mix.right.dt_bias", Hr, 1.0f, 0.f, &w.dt_bias);
            BG_F32(p + "mix.right.norm", Dvr, 0.1f, 1.0f, &w.rnorm);
            BG_GET(p + "mix.right.o", W, Hr * Dvr, amp(Hr * Dvr), 0.f, &a);
            BG_TRY(upload_matrix(a, &w.ro));
            if (R.conv > 1) w.s_rconv = take((int64_t)(R.conv - 1) * C);
            w.s_S = take(Hr * Dr * Dvr);
        }
        w.n_proj = ((int64_t)(stack.size() / (size_t)W) + 31) / 32 * 32; // whole tiles for the tensor-core product
        stack.resize((size_t)(w.n_proj * W), 0.f);
        BG_TRY(upload_matrix(stack, &w.proj));
        if (l.ff > 0) {
            BG_F32(p + "norm2", W, 0.1f, 1.0f, &w.norm2);
            BG_GET(p + "mlp.gate", l.ff, W, aw, 0.f, &a);
            BG_GET(p + "mlp.up", l.ff, W, aw, 0.f, &b);
            a.insert(a.end(), b.begin(), b.end());
            BG_TRY(upload_matrix(a, &w.gate_up));
            BG_F32(p + "mlp.gate.b", l.ff, 0.3f, 0.f, &w.gate_b);
            BG_F32(p + "mlp.up.b", l.ff, 0.3f, 0.f, &w.up_b);
            BG_GET(p + "mlp.down", W, l.ff, amp(l.ff), 0.f, &a);
            BG_TRY(upload_matrix(a, &w.down));
            BG_F32(p + "mlp.down.b", W, 0.3f, 0.f, &w.down_b);
        }
    }
#undef BG_GET
#undef BG_F32
    state_elems_ = st;
    // pages behind the widest window are never read again; one unbounded window keeps everything
    lookback_ = 0;
    bool bounded = n_cache > 0;
    for (const bg_layer_cfg &l : c.layers)
        if (l.type == 1) {
            if (l.left.window <= 0) bounded = false;
            lookback_ = std::max(lookback_, l.left.window);
        }
    if (!bounded) lookback_ = 0;
    return 0;
}

lm_model *begupel_model::create(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err) {
    begupel_model *m = new begupel_model();
    safetensors_file file;
    m->dt_ = opt.dtype;
    if (opt.max_portion > 0) m->max_T_ = opt.max_portion;
    int rc = bg_parse_config(cfg, &m->cfg_, &m->err_);
    if (!rc && !ggb_dtype_size(m->dt_)) rc = -1, m->err_ = "Begupel runs in bfloat16 or float32";
    if (!rc && !opt.random_weights) rc = file.open(dir + "/model.safetensors", &m->err_);
    if (!rc) rc = m->load(opt.random_weights ? nullptr : &file, opt.seed);
    if (rc) {
        if (err) *err = m->err_;
        delete m;
        return nullptr;
    }
    return m;
}

begupel_model::~begupel_model() {
    ggb_sync();
    for (step_graph &g : graphs_) ggb_graph_free(g.graph);
    for (void *p : owned_) ggb_buffer_free(p);
}

std::vector<int64_t> begupel_model::cache_row_elems() const {
    std::vector<int64_t> v;
    for (const bg_layer_cfg &l : cfg_.layers)
        if (l.type == 1) v.push_back(ggb_window_cache_ld(l.left.kv_heads, l.left.dim, l.left.vdim));
    return v;
}

// ------------------------------------------------------------------------------------------------ buffers
int begupel_model::alloc_scratch() {
    const bg_config &c = cfg_;
    const int64_t T = max_T_, W = c.width;
    int64_t npr = 0, ncv = 0, nq = 0, nro = 0, nao = 0, ff = 0;
    int hmax = 1;
    for (size_t li = 0; li < c.layers.size(); li++) {
        const bg_layer_cfg &l = c.layers[li];
        npr = std::max(npr, lw_[li].n_proj);
        if (l.type == 0) {
            nro = std::max(nro, (int64_t)l.heads * l.vdim);
        } else {
            ncv = std::max(ncv, 2 * (int64_t)l.right.kv_heads * l.right.dim + (int64_t)l.right.heads * l.right.vdim);
            nq = std::max(nq, (int64_t)l.left.heads * l.left.dim);
            nao = std::max(nao, (int64_t)l.left.heads * l.left.vdim);
            hmax = std::max(hmax, l.left.heads);
            nro = std::max(nro, (int64_t)l.right.heads * l.right.vdim);
        }
        ff = std::max(ff, (int64_t)l.ff);
    }
    const size_t es = ggb_dtype_size(dt_);
    auto alloc = [&](size_t bytes, void **p) -> int {
        BG_TRY(ggb_buffer_alloc(std::max<size_t>(bytes, 16), p));
        owned_.push_back(*p);
        return 0;
    };
#define BG_ALLOC(ptr, bytes) BG_TRY(alloc((size_t)(bytes), (void **)&(ptr)))
    BG_ALLOC(ids_, T * 4);
    BG_ALLOC(want_, T * 4);
    BG_ALLOC(iota_, T * 4);
    BG_ALLOC(pos0_, 16);
    BG_ALLOC(x_, T * W * 4);
    BG_ALLOC(h_, T * W * es);
    BG_ALLOC(pr_, T * npr * 4);
    BG_ALLOC(cv_, T * ncv * 4);
    BG_ALLOC(qr_, T * nq * 4);
    BG_ALLOC(ao_, T * nao * es);
    BG_ALLOC(wa_, ggb_window_attn_scratch_bytes(hmax));
    BG_ALLOC(ro_, T * nro * 4);
    BG_ALLOC(gd_, T * nro * es);
    BG_ALLOC(ya_, T * W * 4);
    BG_ALLOC(yb_, T * W * 4);
    BG_ALLOC(xd_, T * W * es);
    BG_ALLOC(gu_, T * 2 * ff * 4);
    BG_ALLOC(act_, T * ff * es);
    BG_ALLOC(xw_, T * W * 4);
    BG_ALLOC(hw_, T * W * es);
    BG_ALLOC(logits_, T * (int64_t)c.vocab * 4);
#undef BG_ALLOC
    std::vector<int32_t> iota((size_t)T);
    for (int64_t i = 0; i < T; i++) iota[(size_t)i] = (int32_t)i;
    BG_TRY(ggb_upload(iota_, iota.data(), (size_t)T * 4));
    BG_TRY(ggb_sync());
    return 0;
}

int begupel_model::bind_cache(paged_cache *cache, int64_t max_positions) {
    cache_ = cache;
    max_pos_ = max_positions;
    if ((int)cache_row_elems().size() != cache->n_layers()) return fail(GGB_ERR_ARG, "the cache has another number of layers than the model");
    if (cache->state_elems() < state_elems_) return fail(GGB_ERR_ARG, "the cache keeps less state per sequence than the model needs");
    auto table = [&](const rot_spec &r, const float **out) -> int {
        *out = nullptr;
        if (r.dims <= 0) return 0;
        const std::string k = r.key();
        if (!rot_tables_.count(k)) {
            float *d = nullptr;
            BG_TRY(upload_f32(rot_table(r, max_positions), &d));
            rot_tables_[k] = d;
        }
        *out = rot_tables_[k];
        return 0;
    };
    for (size_t li = 0; li < cfg_.layers.size(); li++)
        if (cfg_.layers[li].type == 1) {
            BG_TRY(table(cfg_.layers[li].left.rot, &lw_[li].cs_k));
            BG_TRY(table(cfg_.layers[li].left.vrot, &lw_[li].cs_v));
        }
    return alloc_scratch();
}

// ------------------------------------------------------------------------------------------------ one portion
int begupel_model::emit(int T, const int32_t *table, float *state, int n_want) {
    const bg_config &c = cfg_;
    const int64_t W = c.width, t = T;
    const int B = cache_->page_size();
    if (c.buckets > 0)
        BG_OP("op_rows", ggb_op_embed_bigram(dt_, embed_, bigram_, ids_, t, W, c.buckets, c.mul_prev, c.mul_cur, pos0_, (int32_t *)state, x_));
    else
        BG_OP("op_rows", ggb_op_embed_rows(dt_, embed_, ids_, t, W, x_));
    for (size_t li = 0; li < c.layers.size(); li++) {
        const bg_layer_cfg &l = c.layers[li];
        const bg_layer_w &w = lw_[li];
        const int64_t N = w.n_proj;
        // h = x + conv(x) in the matrices' type, then every projection of the mixer in one product
        BG_OP("op_conv", ggb_op_causal_conv(dt_, x_, W, t, W, w.canon, std::max(c.taps, 1), 1, 0, state + w.s_canon, nullptr, 0, h_));
        BG_OP("op_linear", ggb_op_linear(dt_, w.proj, N, W, h_, W, t, pr_, N));
        if (l.type == 0) {
            const int H = l.heads, D = l.dim, Dv = l.vdim;
            const int64_t HV = (int64_t)H * Dv;
            BG_OP("op_recurrence", ggb_op_lightning_attn(pr_ + w.o_q, pr_ + w.o_k, pr_ + w.o_v, N, t, H, D, Dv, w.decay, state + w.s_S, ro_, HV));
            BG_OP("op_norm", ggb_op_norm_gate(dt_, ro_, HV, pr_ + w.o_g, N, t, 1, (int)HV, w.mix_norm, (int)HV, c.eps, 0, gd_));
            BG_OP("op_linear", ggb_op_linear(dt_, w.o, W, HV, gd_, HV, t, ya_, W));
            BG_OP("op_residual", ggb_op_group_norm_add(dt_, ya_, 1.0f, nullptr, 0.f, nullptr, w.norm1, c.groups, c.eps, W, t, x_, l.ff ? xd_ : nullptr));
        } else {
            const bg_window_cfg &A = l.left;
            const bg_delta_cfg &R = l.right;
            void *cache = cache_->layer(w.cache_index);
            const int64_t HV = (int64_t)A.heads * A.vdim;
            BG_OP("op_attn_prep", ggb_op_window_qkv_store(dt_, pr_ + w.o_q, pr_ + w.o_k, pr_ + w.o_v, N, t, A.heads, A.kv_heads, A.dim, A.vdim, w.qn,
                                                          w.kn, c.eps, A.rot.dims, w.cs_k, w.cs_v, A.scale, pos0_, table, B, cache, qr_));
            BG_OP("op_attn", ggb_op_window_attn(dt_, qr_, cache, table, B, pos0_, t, A.heads, A.kv_heads, A.dim, A.vdim, A.window, w.cs_v, ao_, wa_));
            BG_OP("op_linear", ggb_op_linear(dt_, w.o, W, HV, ao_, HV, t, ya_, W));
            const int64_t GD = (int64_t)R.kv_heads * R.dim, RV = (int64_t)R.heads * R.vdim, C = 2 * GD + RV;
            BG_OP("op_conv", ggb_op_causal_conv(dt_, pr_ + w.o_rq, N, t, C, w.rconv, R.conv, 0, 1, R.conv > 1 ? state + w.s_rconv : nullptr, cv_, C, nullptr));
            BG_OP("op_recurrence", ggb_op_gated_delta(cv_, cv_ + GD, cv_ + 2 * GD, C, pr_ + w.o_rb, pr_ + w.o_ra, N, t, R.heads, R.kv_heads, R.dim, R.vdim,
                                                      w.A_log, w.dt_bias, state + w.s_S, ro_, RV));
            BG_OP("op_norm", ggb_op_norm_gate(dt_, ro_, RV, pr_ + w.o_rg, N, t, R.heads, R.vdim, w.rnorm, R.vdim, c.eps, 1, gd_));
            BG_OP("op_linear", ggb_op_linear(dt_, w.ro, W, RV, gd_, RV, t, yb_, W));
            BG_OP("op_residual", ggb_op_group_norm_add(dt_, ya_, l.left_scale, yb_, l.right_scale, nullptr, w.norm1, c.groups, c.eps, W, t, x_,
                                                       l.ff ? xd_ : nullptr));
        }
        if (l.ff > 0) {
            BG_OP("op_linear", ggb_op_linear(dt_, w.gate_up, 2 * (int64_t)l.ff, W, xd_, W, t, gu_, 2 * (int64_t)l.ff));
            BG_OP("op_act", ggb_op_glu_bias(dt_, gu_, l.ff, t, w.gate_b, w.up_b, 0, act_));
            BG_OP("op_linear", ggb_op_linear(dt_, w.down, W, l.ff, act_, l.ff, t, ya_, W));
            BG_OP("op_residual", ggb_op_group_norm_add(dt_, ya_, 1.0f, nullptr, 0.f, w.down_b, w.norm2, c.groups, c.eps, W, t, x_, nullptr));
        }
        if (capture_ && cap_) BG_OP("op_rows", ggb_op_gather_rows_f32(x_, iota_, t, W, cap_ + li * (size_t)max_T_ * (size_t)W));
    }
    if (n_want > 0) {
        BG_OP("op_rows", ggb_op_gather_rows_f32(x_, want_, n_want, W, xw_));
        BG_OP("op_norm", ggb_op_group_norm_add(dt_, xw_, 1.0f, nullptr, 0.f, nullptr, final_norm_, c.groups, c.eps, W, n_want, nullptr, hw_));
        BG_OP("op_linear", ggb_op_linear(dt_, head_, c.vocab, W, hw_, W, n_want, logits_, c.vocab));
        if (c.softcap > 0.f) BG_OP("op_act", ggb_op_softcap(logits_, (int64_t)n_want * c.vocab, c.softcap));
    }
    return 0;
}

int begupel_model::forward(const lm_portion &p, const int32_t *want, int n_want) {
    if (!cache_) return fail(GGB_ERR_ARG, "forward before bind_cache");
    if (p.T <= 0 || p.T > max_T_ || n_want < 0 || n_want > p.T || p.pos0 < 0 || p.pos0 + p.T > max_pos_ || !p.state_dev) {
        err_ = "forward: a portion of " + std::to_string(p.T) + " tokens at position " + std::to_string(p.pos0) + " does not fit";
        return GGB_ERR_ARG;
    }
    for (int i = 0; i < p.T; i++)
        if (p.tokens[i] < 0 || p.tokens[i] >= cfg_.vocab) {
            err_ = "forward: token " + std::to_string(p.tokens[i]) + " is outside the vocabulary";
            return GGB_ERR_ARG;
        }
    const int32_t pos0 = (int32_t)p.pos0;
    BG_TRY(ggb_upload(ids_, p.tokens, (size_t)p.T * 4));
    BG_TRY(ggb_upload(pos0_, &pos0, 4));
    if (n_want) BG_TRY(ggb_upload(want_, want, (size_t)n_want * 4));
    const int64_t l0 = ggb_launch_count();
    if (capture_) {
        if (!cap_) {
            void *d = nullptr;
            BG_TRY(ggb_buffer_alloc(cfg_.layers.size() * (size_t)max_T_ * (size_t)cfg_.width * 4, &d));
            owned_.push_back(d);
            cap_ = (float *)d;
        }
        cap_T_ = p.T;
    }
    if (p.T == 1 && use_graphs_ && !capture_ && !getenv("GGB_NO_STEP_GRAPH")) {
        ggb_graph *g = nullptr;
        for (const step_graph &sg : graphs_)
            if (sg.table == p.block_table_dev && sg.state == p.state_dev && sg.n_want == n_want) g = sg.graph;
        if (!g) {
            BG_TRY(ggb_capture_begin());
            const int rc = emit(1, p.block_table_dev, p.state_dev, n_want);
            const int rc2 = ggb_capture_end(&g);
            if (rc) return rc;
            if (rc2) return fail(rc2, "ggb_capture_end");
            if (graphs_.size() >= 32) {
                ggb_graph_free(graphs_.front().graph);
                graphs_.erase(graphs_.begin());
            }
            graphs_.push_back(step_graph{p.block_table_dev, p.state_dev, n_want, g});
        }
        BG_TRY(ggb_graph_launch(g));
    } else {
        BG_TRY(emit(p.T, p.block_table_dev, p.state_dev, n_want));
    }
    kernels_last_ = (int)(ggb_launch_count() - l0);
    return 0;
}

int begupel_model::get_capture(int layer, float *host, int64_t n) const {
    if (!cap_ || layer < 0 || layer >= (int)cfg_.layers.size() || n > (int64_t)cap_T_ * cfg_.width) return GGB_ERR_ARG;
    return ggb_download(host, cap_ + (size_t)layer * (size_t)max_T_ * (size_t)cfg_.width, (size_t)n * 4);
}

namespace {
struct register_begupel {
    register_begupel() { lm_register("Begupel", &begupel_model::create); }
} g_register_begupel;
} // namespace
