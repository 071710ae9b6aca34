// Engine level of the C ABI: continuous batching over the paged KV cache.
// The reference decodes one sequence at a time (ARCHITECTURE.md:376-377); here up to max_seqs
// independent `InferenceSession`-equivalent sequences share every launch. Each scheduler step
// packs one decode row per running sequence plus all prompt rows of newly admitted sequences
// into one ragged batch, so every layer-op is launched once per step.
//
// Block allocation is deterministic: the lowest free block index is handed out first, a
// sequence reserves ceil(max_total_len/16) blocks at admission and returns them before the
// next admission once it has finished.
#include <limits.h>

#include <deque>
#include <map>
#include <set>

#include "model.h"

using namespace ak;

namespace {

struct Seq {
    uint64_t id = 0;
    std::vector<uint32_t> prompt;
    uint32_t max_total = 0;
    std::vector<int32_t> blocks;
    std::vector<uint32_t> generated;
    uint32_t cached = 0;  // tokens whose K/V are in the cache
    int slot = -1;
    bool finished = false;
    bool in_prefill = false;   // admitted, its prompt is not fully in the cache yet
    uint32_t prefilled = 0;    // prompt tokens already scheduled into the cache
};

}  // namespace

struct ak_engine {
    ak_ctx* ctx = nullptr;
    ak_weights* w = nullptr;
    ak_engine_config cfg{};
    Runner runner;
    std::set<int32_t> free_blocks;
    std::vector<Seq*> slots;     // running sequence per slot (nullptr = free)
    std::deque<Seq*> waiting;
    std::map<uint64_t, Seq*> all;
    uint64_t next_id = 1;
    ak_engine_stats stats{};
    unsigned long long launch_base = 0;
    double launch_host_base = 0.0;   // the runner's cumulative launch time at the last ak_engine_reset_stats
    // a step that has been launched and whose tokens have not been read yet
    struct Pending {
        bool active = false;
        uint32_t bank = 0;
        std::vector<std::pair<Seq*, uint32_t>> fill;  // (sequence, index into its `generated`), slot = seq->slot at launch
        std::vector<uint32_t> fill_slot;
        bool any_decode = false;
        bool has_prefill = false;
        uint64_t attn_bytes = 0;
        uint64_t step_bytes = 0;
    } pending;
    uint64_t weight_bytes = 0;   // bytes of every tensor a decode step reads in full (all but the embedding table)
    uint64_t step_index = 0;
    std::deque<Seq*> prefill_queue;   // admitted sequences whose prompt is not fully scheduled, in admission order
    uint32_t chunk_rows = 0;          // prompt rows per step while others decode (0 = whole prompts only)
    bool async_ok() const { return cfg.async_steps != 0 && cfg.stop_on_eos == 0; }
};

// Wait for the step in flight and write its tokens into their sequences.
static int collect(ak_engine* e) {
    ak_engine::Pending& p = e->pending;
    if (!p.active) return AK_OK;
    Runner& r = e->runner;
    int rc = r.wait_bank(p.bank);
    if (rc) return rc;
    const uint32_t cur = r.bank();
    r.set_bank(p.bank);
    const uint32_t* sampled = r.h_sampled();
    const ak_model_config& mc = e->w->cfg;
    for (size_t i = 0; i < p.fill.size(); i++) {
        Seq* s = p.fill[i].first;
        const uint32_t tok = sampled[p.fill_slot[i]];
        s->generated[p.fill[i].second] = tok;
        if (e->cfg.stop_on_eos && tok == mc.eos_token) s->finished = true;
    }
    const float step_ms = e->cfg.attn_timing ? r.last_step_gpu_ms() : 0.0f;
    e->stats.step_gpu_ms_total += step_ms;
    // the roofline sample: decode-only steps (in an admission step the prompt's kernels run beside the attention)
    if (e->cfg.attn_timing && p.any_decode && !p.has_prefill) {
        if (step_ms > 0.0f) {
            e->stats.decode_step_gpu_ms_total += step_ms;
            e->stats.decode_steps_timed++;
            e->stats.decode_step_bytes_total += p.step_bytes;
        }
        float ms = r.last_attn_ms();
        if (ms > 0.0f) {
            e->stats.attn_ms_total += ms;
            e->stats.attn_launches_timed++;
            e->stats.attn_bytes_total += p.attn_bytes;
        }
    }
    r.set_bank(cur);
    p.active = false;
    return AK_OK;
}

static void release(ak_engine* e, Seq* s) {
    for (int32_t b : s->blocks) e->free_blocks.insert(b);
    // the block list is kept for ak_engine_block_table on finished sequences
    if (s->slot >= 0) e->slots[s->slot] = nullptr;
    s->slot = -1;
}

extern "C" {

int ak_engine_create(ak_ctx* ctx, ak_weights* w, const ak_engine_config* cfg, ak_engine** out) {
    AK_REQUIRE(ctx && w && cfg && out, AK_ERR_INVALID_ARG, "ak_engine_create: null pointer");
    AK_REQUIRE(cfg->max_seqs >= 1 && cfg->max_seq_len >= 1, AK_ERR_INVALID_ARG, "ak_engine_create: max_seqs and max_seq_len must be >= 1");
    AK_REQUIRE(cfg->block_size == 16 || cfg->block_size == 0, AK_ERR_UNSUPPORTED, "ak_engine_create: block_size must be 16");
    ak_engine* e = new ak_engine();
    e->ctx = ctx;
    e->w = w;
    e->cfg = *cfg;
    e->cfg.block_size = 16;
    const uint32_t mb = (cfg->max_seq_len + 15) / 16;
    if (e->cfg.kv_blocks == 0) e->cfg.kv_blocks = cfg->max_seqs * mb;
    if (e->cfg.max_batch_tokens < cfg->max_seqs + 1) {
        // default step budget: every slot may be (re)filled in one step, capped at 32k prompt rows
        uint64_t pf = (uint64_t)cfg->max_seqs * cfg->max_seq_len;
        if (pf > 32768) pf = 32768;
        if (pf < cfg->max_seq_len) pf = cfg->max_seq_len;
        e->cfg.max_batch_tokens = cfg->max_seqs + (uint32_t)pf;
    }
    int rc = e->runner.init(ctx, w, cfg->max_seqs, cfg->max_seq_len, e->cfg.kv_blocks, e->cfg.max_batch_tokens - cfg->max_seqs);
    if (rc) {
        delete e;
        return rc;
    }
    e->chunk_rows = e->runner.chunked_prefill_supported() ? cfg->prefill_chunk_rows : 0;
    if (e->chunk_rows > e->runner.max_prefill_tokens()) e->chunk_rows = e->runner.max_prefill_tokens();
    e->runner.enable_attn_timing(cfg->attn_timing != 0);
    e->runner.set_keep_logits(false);
    for (const auto& pr : w->params)
        if (pr.kind != 1) e->weight_bytes += pr.llen * (pr.kind == 0 ? 4 : (w->dtype == AK_F32 ? 4 : 2));
    for (uint32_t b = 0; b < e->cfg.kv_blocks; b++) e->free_blocks.insert((int32_t)b);
    e->slots.assign(cfg->max_seqs, nullptr);
    *out = e;
    return AK_OK;
}

int ak_engine_destroy(ak_engine* e) {
    if (!e) return AK_OK;
    collect(e);
    for (auto& kv : e->all) delete kv.second;
    delete e;
    return AK_OK;
}

int ak_engine_submit(ak_engine* e, const uint32_t* prompt, uint32_t n, uint32_t max_total_len, uint64_t* seq_id) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_submit: null engine");
    AK_REQUIRE(n != 0, AK_EMPTY_PROMPT, "prompt is empty");
    AK_REQUIRE(prompt, AK_ERR_INVALID_ARG, "ak_engine_submit: null prompt");
    AK_REQUIRE(n <= e->cfg.max_seq_len && n <= e->runner.max_prefill_tokens(), AK_PROMPT_TOO_LONG,
               "prompt is %u tokens, context window is %u (step budget %u)", n, e->cfg.max_seq_len, e->runner.max_prefill_tokens());
    if (max_total_len > e->cfg.max_seq_len) max_total_len = e->cfg.max_seq_len;
    AK_REQUIRE(max_total_len > n, AK_CONTEXT_FULL, "context window is full (%u tokens)", max_total_len);
    // a sequence reserves all of its blocks at admission: one that needs more than the pool holds could never start
    AK_REQUIRE((max_total_len + 15) / 16 <= e->cfg.kv_blocks, AK_CONTEXT_FULL,
               "sequence of up to %u tokens needs %u KV blocks, the pool holds %u", max_total_len, (max_total_len + 15) / 16, e->cfg.kv_blocks);
    Seq* s = new Seq();
    s->id = e->next_id++;
    s->prompt.assign(prompt, prompt + n);
    s->max_total = max_total_len;
    e->all[s->id] = s;
    e->waiting.push_back(s);
    if (seq_id) *seq_id = s->id;
    return AK_OK;
}

int ak_engine_step(ak_engine* e, uint32_t* n_running, uint32_t* n_waiting) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_step: null engine");
    Runner& r = e->runner;
    const uint32_t S = e->cfg.max_seqs;
    const ak_model_config& mc = e->w->cfg;
    const unsigned long long launches0 = g_launch_count;
    // Without async steps the previous step's tokens decide who has finished: read them first.
    // With async steps sequence ends depend on lengths only, so this step is planned and launched
    // while the previous one still runs, and the previous one's tokens are read afterwards.
    if (!e->async_ok()) { int rc0 = collect(e); if (rc0) return rc0; }
    r.set_bank(e->async_ok() ? (uint32_t)(e->step_index & 1u) : 0u);

    // 1. retire sequences that finished in the previous step (their blocks go back first)
    for (uint32_t i = 0; i < S; i++)
        if (e->slots[i] && e->slots[i]->finished) release(e, e->slots[i]);

    // 2. admit waiting sequences in arrival order into the lowest free slots; their prompts join the prefill queue
    while (!e->waiting.empty()) {
        Seq* s = e->waiting.front();
        int slot = -1;
        for (uint32_t i = 0; i < S; i++)
            if (!e->slots[i]) { slot = (int)i; break; }
        const uint32_t need = (s->max_total + 15) / 16;
        if (slot < 0 || e->free_blocks.size() < need) break;
        e->waiting.pop_front();
        s->slot = slot;
        e->slots[slot] = s;
        s->blocks.clear();
        for (uint32_t b = 0; b < need; b++) {
            auto it = e->free_blocks.begin();
            s->blocks.push_back(*it);
            e->free_blocks.erase(it);
        }
        s->in_prefill = true;
        s->prefilled = 0;
        e->prefill_queue.push_back(s);
    }

    // 3. choose the prompt rows of this step.
    // Whole prompts (as many as fit the step budget) when nobody is decoding or a lot of prompt is pending. Otherwise
    // chunks: while other sequences decode, a prompt is prefilled `chunk_rows` rows per step, so that decode rows and
    // prompt rows together stay within ONE 128-row tile of every projection and the prompt rides in the decode
    // launches; its sequence samples its first token in the step that holds its last chunk. Chunk boundaries depend on
    // the prompt alone, and a row's arithmetic does not depend on which rows share its launch.
    bool decoding_now = false;
    for (uint32_t i = 0; i < S; i++) decoding_now |= (e->slots[i] && !e->slots[i]->finished && !e->slots[i]->in_prefill);
    uint64_t pending_rows = 0;
    for (Seq* s : e->prefill_queue) pending_rows += s->prompt.size() - s->prefilled;
    const bool chunk_mode = e->chunk_rows > 0 && decoding_now && pending_rows > 0 && pending_rows <= 8ull * e->chunk_rows;
    const uint32_t budget = chunk_mode ? e->chunk_rows : r.max_prefill_tokens();
    struct Work { Seq* s; uint32_t c0, n; bool last; };
    std::vector<Work> work;
    uint32_t pf_rows = 0;
    for (Seq* s : e->prefill_queue) {
        const uint32_t left = (uint32_t)s->prompt.size() - s->prefilled;
        uint32_t take = left;
        if (chunk_mode) { if (take > budget - pf_rows) take = budget - pf_rows; }
        else if (pf_rows + take > budget) break;     // whole prompts only: the next one waits for the next step
        if (take == 0) break;
        work.push_back({s, s->prefilled, take, take == left});
        pf_rows += take;
        if (pf_rows >= budget) break;
    }

    // 4. describe the step: decode rows by slot, then the prompt rows
    RowInfo* rows = r.h_rows();
    int32_t* kv = r.h_kv_lens();
    int32_t* outr = r.h_out_rows();
    bool any_decode = false;
    uint32_t max_kv = 1;
    uint64_t attn_bytes = 0;
    const uint64_t esz = e->w->dtype == AK_F32 ? 4 : 2;
    uint32_t n_dec = 0;
    for (uint32_t i = 0; i < S; i++) {
        Seq* s = e->slots[i];
        if (s && !s->finished) {
            // every bank of the descriptor carries its own copy of the tables: refresh the live ones
            int32_t* bt = r.h_block_table(i);
            const uint32_t nb = (uint32_t)s->blocks.size();
            for (uint32_t b = 0; b < r.max_blocks(); b++) bt[b] = b < nb ? s->blocks[b] : 0;
        }
        if (s && !s->finished && !s->in_prefill) {
            const uint32_t pos = s->cached;
            rows[i] = {-(int32_t)(i + 1), (int32_t)pos, s->blocks[pos / 16] * 16 + (int32_t)(pos % 16), (int32_t)i};
            kv[i] = (int32_t)(pos + 1);
            outr[i] = (int32_t)i;
            any_decode = true;
            n_dec++;
            if (pos + 1 > max_kv) max_kv = pos + 1;
            const uint64_t qd = r.local_qdim();  // this rank's share of the heads
            attn_bytes += (uint64_t)(pos + 1) * qd * 2 * esz + qd * 2 * esz + (uint64_t)((pos + 16) / 16) * 4;
        } else {
            rows[i] = {INT_MIN, -1, -1, (int32_t)i};
            kv[i] = 0;
            outr[i] = -1;
        }
    }
    uint32_t row = S, max_pf = 0;
    int32_t* cu = r.h_pf_cu();
    int32_t* pfs = r.h_pf_slot();
    int32_t* p0 = r.h_pf_pos0();
    cu[0] = 0;
    for (size_t a = 0; a < work.size(); a++) {
        Seq* s = work[a].s;
        const uint32_t c0 = work[a].c0, n = work[a].n;
        for (uint32_t j = 0; j < n; j++) {
            const uint32_t pos = c0 + j, t = s->prompt[pos];
            rows[row + j] = {t > 0x7fffffffu ? INT_MAX : (int32_t)t, (int32_t)pos, s->blocks[pos / 16] * 16 + (int32_t)(pos % 16), s->slot};
        }
        row += n;
        cu[a + 1] = (int32_t)(row - S);
        pfs[a] = s->slot;
        p0[a] = (int32_t)c0;
        // the sequence samples its first token from the last row of its last chunk
        outr[s->slot] = work[a].last ? (int32_t)(row - 1) : -1;
        if (n > max_pf) max_pf = n;
    }
    if (!any_decode && work.empty()) {
        int rcf = collect(e);  // nothing to launch: make the last step's tokens visible
        if (rcf) return rcf;
        if (n_running) *n_running = 0;
        if (n_waiting) *n_waiting = (uint32_t)e->waiting.size();
        return AK_OK;
    }

    // 5. launch
    int rc;
    const bool graph = e->cfg.use_cuda_graph != 0;
    if (graph) rc = r.run_graph(pf_rows, (uint32_t)work.size(), max_pf);
    else rc = r.run(pf_rows, (uint32_t)work.size(), max_pf, any_decode, max_kv);
    if (rc) return rc;
    rc = r.mark_done();
    if (rc) return rc;

    // 6. advance the sequences (token values are filled in when the step is collected)
    ak_engine::Pending now;
    now.active = true;
    now.bank = r.bank();
    now.any_decode = any_decode;
    now.has_prefill = pf_rows != 0;
    now.attn_bytes = attn_bytes;
    // per layer: the attention launch's bytes plus one appended K and V row per sequence; per step: the weights
    // and one embedding row per sequence
    now.step_bytes = e->weight_bytes + (uint64_t)n_dec * mc.dim * esz +
                     (uint64_t)mc.num_layers * (attn_bytes + (uint64_t)n_dec * 2 * r.local_qdim() * esz);
    auto emit_token = [&](Seq* s) {
        now.fill.emplace_back(s, (uint32_t)s->generated.size());
        now.fill_slot.push_back((uint32_t)s->slot);
        s->generated.push_back(0);
        if (s->prompt.size() + s->generated.size() >= s->max_total) s->finished = true;
    };
    for (uint32_t i = 0; i < S; i++) {
        Seq* s = e->slots[i];
        if (!s || s->finished || s->in_prefill) continue;
        s->cached++;
        emit_token(s);
    }
    for (const Work& wk : work) {
        wk.s->prefilled += wk.n;
        if (!wk.last) continue;
        wk.s->in_prefill = false;
        wk.s->cached = (uint32_t)wk.s->prompt.size();
        emit_token(wk.s);
    }
    while (!e->prefill_queue.empty() && !e->prefill_queue.front()->in_prefill) e->prefill_queue.pop_front();
    uint32_t running = 0;
    for (uint32_t i = 0; i < S; i++) if (e->slots[i] && !e->slots[i]->finished) running++;
    // the previous step (other bank) has had this step's host work to finish in: read its tokens now
    rc = collect(e);
    if (rc) return rc;
    e->pending = std::move(now);
    e->step_index++;
    if (!e->async_ok()) {
        rc = collect(e);
        if (rc) return rc;
        // an end-of-sequence token may have finished sequences that the length rule left running
        running = 0;
        for (uint32_t i = 0; i < S; i++) if (e->slots[i] && !e->slots[i]->finished) running++;
    }
    e->stats.steps++;
    e->stats.decode_tokens += n_dec;
    e->stats.prefill_tokens += pf_rows;
    if (graph) e->stats.graph_launches++; else e->stats.eager_steps++;
    e->stats.kernel_launches += (g_launch_count - launches0);
    e->stats.h2d_bytes = r.h2d_bytes;
    e->stats.launch_host_ms_total = r.launch_host_ms - e->launch_host_base;
    e->stats.d2h_bytes = r.d2h_bytes;
    if (n_running) *n_running = running;
    if (n_waiting) *n_waiting = (uint32_t)e->waiting.size();
    return AK_OK;
}

int ak_engine_run(ak_engine* e, uint64_t max_steps, uint64_t* steps_done) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_run: null engine");
    uint64_t n = 0;
    for (;;) {
        if (max_steps && n >= max_steps) break;
        uint32_t running = 0, waiting = 0;
        const uint64_t launched0 = e->stats.steps;
        int rc = ak_engine_step(e, &running, &waiting);
        if (rc) return rc;
        n++;
        if (running == 0 && waiting == 0) break;
        // nothing runs, nothing was launched, yet sequences wait: no later step can admit them either
        AK_REQUIRE(!(running == 0 && e->stats.steps == launched0), AK_ERR_INVALID_ARG,
                   "ak_engine_run: %u waiting sequence(s) can never be admitted (KV pool or step budget too small)", waiting);
    }
    int rc = collect(e);
    if (rc) return rc;
    if (steps_done) *steps_done = n;
    return AK_OK;
}

int ak_engine_poll(ak_engine* e, uint64_t seq_id, uint32_t* out, uint32_t cap, uint32_t* n_out, int* finished) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_poll: null engine");
    { int rcf = collect(e); if (rcf) return rcf; }
    auto it = e->all.find(seq_id);
    AK_REQUIRE(it != e->all.end(), AK_ERR_NOT_FOUND, "ak_engine_poll: unknown sequence %llu", (unsigned long long)seq_id);
    Seq* s = it->second;
    uint32_t n = (uint32_t)s->generated.size();
    if (out)
        for (uint32_t i = 0; i < n && i < cap; i++) out[i] = s->generated[i];
    if (n_out) *n_out = n;
    if (finished) *finished = s->finished ? 1 : 0;
    return AK_OK;
}

int ak_engine_block_table(ak_engine* e, uint64_t seq_id, int32_t* out, uint32_t cap, uint32_t* n_out) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_block_table: null engine");
    { int rcf = collect(e); if (rcf) return rcf; }
    auto it = e->all.find(seq_id);
    AK_REQUIRE(it != e->all.end(), AK_ERR_NOT_FOUND, "ak_engine_block_table: unknown sequence %llu", (unsigned long long)seq_id);
    Seq* s = it->second;
    uint32_t n = (uint32_t)s->blocks.size();
    if (out)
        for (uint32_t i = 0; i < n && i < cap; i++) out[i] = s->blocks[i];
    if (n_out) *n_out = n;
    return AK_OK;
}

int ak_engine_clear_finished(ak_engine* e) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_clear_finished: null engine");
    { int rcf = collect(e); if (rcf) return rcf; }
    for (auto it = e->all.begin(); it != e->all.end();) {
        Seq* s = it->second;
        if (s->finished) {
            if (s->slot >= 0) release(e, s);
            delete s;
            it = e->all.erase(it);
        } else {
            ++it;
        }
    }
    return AK_OK;
}

int ak_engine_get_stats(ak_engine* e, ak_engine_stats* out) {
    AK_REQUIRE(e && out, AK_ERR_INVALID_ARG, "ak_engine_get_stats: null pointer");
    { int rcf = collect(e); if (rcf) return rcf; }
    *out = e->stats;
    return AK_OK;
}
int ak_engine_reset_stats(ak_engine* e) {
    AK_REQUIRE(e, AK_ERR_INVALID_ARG, "ak_engine_reset_stats: null engine");
    { int rcf = collect(e); if (rcf) return rcf; }
    e->stats = ak_engine_stats{};
    e->launch_host_base = e->runner.launch_host_ms;
    return AK_OK;
}

}  // extern "C"
