// AKV3 checkpoint reader: lets real akasha-core checkpoints drive this backend.
// Format (src/nn/checkpoint.rs:18-36, 65-95; bincode 1.x fixed-int little-endian, written by
// hand there too): magic "AKV3"; u32 vocab_size, u32 dim, u32 num_heads, u64 num_layers,
// u32 seq_len, u32 ffn_hidden, u64 train_step, u32 schedule_step; u64 tensor count, then per
// tensor u64 length + f32[length] in `ModelWeights::params()` order; then the AdamW moments
// (u64 count, (m, v) pairs), which inference ignores. `load` (checkpoint.rs:98-161) checks the
// architecture and every tensor length before copying; so does this reader.
#include <stdio.h>
#include <string.h>

#include <vector>

#include "model.h"

using namespace ak;

namespace {

struct Header {
    uint32_t vocab, dim, heads;
    uint64_t layers;
    uint32_t seq_len, ffn;
    uint64_t train_step;
    uint32_t schedule_step;
    uint64_t n_params;
};

bool rd(FILE* f, void* p, size_t n) { return fread(p, 1, n, f) == n; }

int read_header(FILE* f, const char* path, Header* h) {
    char magic[4];
    AK_REQUIRE(rd(f, magic, 4) && memcmp(magic, "AKV3", 4) == 0, AK_ERR_INVALID_ARG, "%s is not a v3 checkpoint (magic AKV3 missing)", path);
    bool ok = rd(f, &h->vocab, 4) && rd(f, &h->dim, 4) && rd(f, &h->heads, 4) && rd(f, &h->layers, 8) && rd(f, &h->seq_len, 4) &&
              rd(f, &h->ffn, 4) && rd(f, &h->train_step, 8) && rd(f, &h->schedule_step, 4) && rd(f, &h->n_params, 8);
    AK_REQUIRE(ok, AK_ERR_INVALID_ARG, "%s: truncated checkpoint header", path);
    return AK_OK;
}

}  // namespace

extern "C" {

int ak_akv3_read_header(const char* path, ak_model_config* cfg_out, uint64_t* train_step_out) {
    AK_REQUIRE(path && cfg_out, AK_ERR_INVALID_ARG, "ak_akv3_read_header: null pointer");
    FILE* f = fopen(path, "rb");
    AK_REQUIRE(f, AK_ERR_NOT_FOUND, "cannot open %s", path);
    Header h{};
    int rc = read_header(f, path, &h);
    fclose(f);
    if (rc) return rc;
    cfg_out->vocab_size = h.vocab;
    cfg_out->dim = h.dim;
    cfg_out->num_heads = h.heads;
    cfg_out->num_layers = (uint32_t)h.layers;
    cfg_out->seq_len = h.seq_len;
    cfg_out->ffn_hidden = h.ffn;
    cfg_out->norm_eps = 1e-5f;              // ModelConfig::new (src/config.rs:25)
    cfg_out->eos_token = h.vocab ? h.vocab - 1 : 0;  // src/config.rs:27-28
    if (train_step_out) *train_step_out = h.train_step;
    return AK_OK;
}

int ak_weights_load_akv3(ak_weights* w, const char* path, uint64_t* train_step_out) {
    AK_REQUIRE(w && path, AK_ERR_INVALID_ARG, "ak_weights_load_akv3: null pointer");
    FILE* f = fopen(path, "rb");
    AK_REQUIRE(f, AK_ERR_NOT_FOUND, "cannot open %s", path);
    Header h{};
    int rc = read_header(f, path, &h);
    if (rc) { fclose(f); return rc; }
    const ak_model_config& c = w->cfg;
    if (h.vocab != c.vocab_size || h.dim != c.dim || h.heads != c.num_heads || h.layers != c.num_layers || h.ffn != c.ffn_hidden) {
        fclose(f);
        set_error("checkpoint architecture mismatch: file (%u, %u, %u, %llu, %u) vs model (%u, %u, %u, %u, %u) "
                  "(vocab_size, dim, num_heads, num_layers, ffn_hidden)",
                  h.vocab, h.dim, h.heads, (unsigned long long)h.layers, h.ffn, c.vocab_size, c.dim, c.num_heads, c.num_layers, c.ffn_hidden);
        return AK_ERR_INVALID_ARG;
    }
    const uint64_t expect = ak_weights_param_count(w);
    if (h.n_params != expect) {
        fclose(f);
        set_error("checkpoint has %llu parameter tensors, model expects %llu", (unsigned long long)h.n_params, (unsigned long long)expect);
        return AK_ERR_INVALID_ARG;
    }
    std::vector<float> buf;
    for (uint32_t i = 0; i < (uint32_t)expect; i++) {
        uint64_t len = 0;
        const uint64_t want = ak_weights_param_len(w, i);
        if (!rd(f, &len, 8)) { fclose(f); set_error("%s: truncated at tensor %u", path, i); return AK_ERR_INVALID_ARG; }
        if (len != want) {
            fclose(f);
            set_error("checkpoint tensor %u has %llu elements, model expects %llu", i, (unsigned long long)len, (unsigned long long)want);
            return AK_ERR_INVALID_ARG;
        }
        buf.resize(len);
        if (!rd(f, buf.data(), len * 4)) { fclose(f); set_error("%s: truncated inside tensor %u", path, i); return AK_ERR_INVALID_ARG; }
        rc = ak_weights_set_param(w, i, buf.data(), len);
        if (rc) { fclose(f); return rc; }
    }
    fclose(f);  // the optimizer moments that follow are not needed for inference
    if (train_step_out) *train_step_out = h.train_step;
    return AK_OK;
}

}  // extern "C"
