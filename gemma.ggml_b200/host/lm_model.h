// lm_model.h — what the serving engine (lm_engine) needs from a model, and the registry that maps the architecture
// name of a model folder's config.json to the class that runs it.  A model declares how many numbers per position
// each of its caching layers keeps; the engine's paged cache (seq_cache.h) owns that memory and hands the model a
// sequence's page table for every forward call.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "json_min.h"

class paged_cache;

// one portion of one sequence: T tokens at positions pos0 .. pos0 + T - 1, pages already reserved
struct lm_portion {
    const int32_t *tokens = nullptr;
    int T = 0;
    int64_t pos0 = 0;
    const int32_t *block_table_dev = nullptr; // device int32 [pages of the sequence]
    float *state_dev = nullptr;               // the sequence's state block (state_elems() fp32 numbers), or null
};

class lm_model {
  public:
    virtual ~lm_model() {}
    virtual const char *architecture() const = 0;
    virtual int vocab() const = 0;
    virtual int dtype() const = 0; // GGB_TYPE_BF16 or GGB_TYPE_F32: storage type of matrices, activations and cache rows
    // numbers per position of every caching layer (empty: the model keeps no per-position state in the paged cache)
    virtual std::vector<int64_t> cache_row_elems() const = 0;
    // called once, before the first forward: the cache the model reads and writes, and the longest sequence it will see
    virtual int bind_cache(paged_cache *cache, int64_t max_positions) = 0;
    // fp32 numbers of state a sequence carries beside its cache rows (recurrent state, convolution tails, the previous
    // token); the cache keeps one zero-initialised block per sequence slot and hands it to forward()
    virtual int64_t state_elems() const { return 0; }
    // how many positions back the farthest-looking caching layer reads (0: unbounded): the engine gives back the pages
    // before that while the sequence lives
    virtual int64_t cache_lookback() const { return 0; }
    virtual int max_live_sequences() const { return 0; } // 0: as many as the engine has slots
    virtual int max_portion() const = 0; // most tokens one forward call takes; the engine cuts longer portions
    // runs the portion from the state earlier portions left in the cache; the logits of rows want[0 .. n_want) of the
    // portion stay on the device: logits_dev() = fp32 [n_want][vocab]
    virtual int forward(const lm_portion &p, const int32_t *want, int n_want) = 0;
    virtual const float *logits_dev() const = 0;
    virtual std::string last_error() const = 0;
    // introspection, optional: the residual stream after every layer of the last portion (fp32 [layers][T][width]),
    // one-token steps as replayed CUDA graphs or eager launches, launch count of the last forward, bytes of weights
    virtual int set_capture(bool) { return -1; }
    virtual int get_capture(int /*layer*/, float * /*host*/, int64_t /*n*/) const { return -1; }
    virtual int set_use_graphs(bool) { return -1; }
    virtual int kernels_last_forward() const { return 0; }
    virtual size_t weight_bytes() const { return 0; }
};

struct lm_load_options {
    int dtype = 30;           // GGB_TYPE_BF16
    int64_t max_tokens = 0;   // most tokens live sequences hold together
    int max_portion = 0;      // 0: the model's default
    bool random_weights = false; // no weight file: numbers generated from `seed` (throughput runs and tests of sizes)
    uint64_t seed = 0;
};

// factory: model folder (config.json parsed into cfg) -> model, or nullptr with *err set
typedef lm_model *(*lm_factory)(const std::string &dir, const json_value &cfg, const lm_load_options &opt, std::string *err);
void lm_register(const char *architecture, lm_factory f);
std::vector<std::string> lm_architectures();
// reads dir/config.json, looks its "architecture" up in the registry and builds the model
lm_model *lm_load(const std::string &dir, const lm_load_options &opt, std::string *err);
// the same from a configuration given as text (dir may be empty with opt.random_weights)
lm_model *lm_load_config(const std::string &config_text, const std::string &dir, const lm_load_options &opt, std::string *err);
