// TEST-ONLY harness: runs the per-word codec core (cubit_b200/csrc/codec_core.cuh, the text the
// CUDA kernels are compiled from) as plain C++ over the host copy of the flat table, so the
// flat-table logic can be compared with the oracle on a machine without a GPU.  It is not
// linked into, loaded by, or reachable from the product library.
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../cubit_b200/csrc/codec_core.cuh"
#include "../../cubit_b200/csrc/flat_table.hpp"
#include "../../cubit_b200/csrc/isa_table.hpp"

using namespace cubit;

struct Mirror {
    IsaTable table;
    FlatTable flat;
    FlatView view;
};

static thread_local std::string g_err;

template <typename Fn>
static void pfor(uint64_t n, int threads, Fn fn) {
    if (threads <= 1 || n < 4096) { fn(0, n); return; }
    std::vector<std::thread> th;
    for (int k = 0; k < threads; ++k)
        th.emplace_back([=] { fn(n * (uint64_t)k / threads, n * (uint64_t)(k + 1) / threads); });
    for (auto& t : th) t.join();
}

extern "C" {
const char* mir_last_error() { return g_err.c_str(); }
void* mir_load(const char* path) {
    try {
        Mirror* m = new Mirror;
        m->table = IsaTable::from_file(path);
        m->flat = FlatTable::compile(m->table);
        m->view = FlatView{m->flat.blob.data(), m->flat.at};
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void* mir_load_text(const char* text, uint64_t len) {
    try {
        Mirror* m = new Mirror;
        m->table = IsaTable::from_json_text(std::string(text, len));
        m->flat = FlatTable::compile(m->table);
        m->view = FlatView{m->flat.blob.data(), m->flat.at};
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void mir_free(void* h) { delete (Mirror*)h; }
// out[0..9]: keys, variants, buckets, largest bucket, nodes, child refs, leaves, classes, largest leaf, depth;
// out[10..11]: hot bytes, total bytes of the table blob
void mir_info(void* h, uint32_t* out) {
    Mirror* m = (Mirror*)h;
    const FlatTable& f = m->flat;
    const uint32_t v[12] = {f.n_keys, (uint32_t)f.meta.size(), f.n_buckets, f.max_bucket, (uint32_t)(f.nodes.size() / NR_WORDS),
                            (uint32_t)f.children.size(), f.n_leaves, (uint32_t)(f.classes.size() / CR_WORDS),
                            f.max_leaf_classes, f.max_depth, f.at.hot_words * 4, f.at.total_words * 4};
    for (int i = 0; i < 12; ++i) out[i] = v[i];
}
// The compiled table blob and its section offsets (BlobLayout as 31 u32).
void mir_blob(void* h, const uint32_t** blob, uint32_t* layout_words) {
    Mirror* m = (Mirror*)h;
    *blob = m->flat.blob.data();
    static_assert(sizeof(BlobLayout) == 31 * sizeof(uint32_t), "layout size");
    memcpy(layout_words, &m->flat.at, sizeof(BlobLayout));
}
// Per word: classes in its leaf, classes that match, tree steps walked (for tuning).
void mir_leaf_stats(void* h, const uint32_t* words, uint64_t n, uint8_t* n_classes, uint8_t* n_match, uint8_t* depth) {
    const Mirror* m = (const Mirror*)h;
    const FlatView& t = m->view;
    for (uint64_t i = 0; i < n; ++i) {
        const uint32_t c0 = words[4 * i], c1 = words[4 * i + 1], c2 = words[4 * i + 2];
        uint32_t start = 0, count = 0, steps = 0;
        uint32_t ref = t.cold[t.at.dir + (c0 & 0xFFFu)];
        if (ref) {
            while (!(ref & REF_LEAF)) {
                ++steps;
                const uint32_t* na = t.cold + t.at.nodes[0] + ref_index(ref) * 4;
                const uint32_t* nb = t.cold + t.at.nodes[1] + ref_index(ref) * 4;
                uint32_t f = (c2 & na[0]) * na[1];
                if (ref & REF_WIDE) f += (c0 & nb[0]) * nb[2] + (c1 & nb[1]) * nb[3];
                ref = t.cold[t.at.children + na[2] + (f >> na[3])];
            }
            start = ref_index(ref); count = ref_count(ref);
        }
        uint32_t matches = 0;
        for (uint32_t k = 0; k < count; ++k)
            { uint32_t fl; matches += class_match<HotPlain>(t, start + k, c0, c1, c2, &fl) != 3; }
        n_classes[i] = (uint8_t)count; n_match[i] = (uint8_t)matches; depth[i] = (uint8_t)steps;
    }
}
// Per word: the choice flag the rules ask for (0 none) and whether the top candidate already has it.
void mir_rule_stats(void* h, const uint32_t* words, uint64_t n, uint32_t* need_out, uint8_t* first_has) {
    const Mirror* m = (const Mirror*)h;
    const FlatView& t = m->view;
    for (uint64_t i = 0; i < n; ++i) {
        const uint32_t c0 = words[4 * i], c1 = words[4 * i + 1], c2 = words[4 * i + 2];
        need_out[i] = 0; first_has[i] = 0;
        uint32_t start, count;
        if (find_leaf<HotPlain>(t, c0, c1, c2, &start, &count) != ST_OK) continue;
        uint32_t first_key = 0xFFFFFFFFu, first_fl = 0, any = 0;
        for (uint32_t k = 0; k < count; ++k) {
            uint32_t fl;
            const uint32_t prio = class_match<HotPlain>(t, start + k, c0, c1, c2, &fl);
            if (prio == 3) continue;
            const uint32_t r = (start + k) * 4;
            const Quad q2 = HotPlain::q(t, t.at.classes[2] + r), q3 = HotPlain::q(t, t.at.classes[3] + r);
            const uint32_t key = (q2.x & ~KEY_WITHIN) | dynamic_key(q3, prio, c0, c1, c2);
            any |= fl;
            if (key < first_key) { first_key = key; first_fl = q2.y; }
        }
        if (first_key == 0xFFFFFFFFu) continue;
        const uint32_t need = choose_rule(any & 0xFFFF, first_fl, c0, c1, c2);
        need_out[i] = need; first_has[i] = (first_fl & need) != 0;
    }
}
// Per word: how many classes the ranking loop has to compare (0: decided by static order alone).
void mir_word_meta(void* h, const uint32_t* words, uint64_t n, uint32_t* max_reg, uint32_t* barriers, uint8_t* is_exit) {
    const Mirror* m = (const Mirror*)h;
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t ex;
        word_meta<HotPlain>(m->view, words[4 * i], words[4 * i + 1], words[4 * i + 2], &max_reg[i], &barriers[i], &ex);
        is_exit[i] = (uint8_t)ex;
    }
}
void mir_decode_batch(void* h, const uint32_t* words, uint64_t n, uint16_t* form, uint32_t* slots, uint32_t* ctrl, int threads) {
    const Mirror* m = (const Mirror*)h;
    pfor(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint32_t f, c, s[8];
            decode_word<HotPlain>(m->view, words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3], &f, s, &c);
            form[i] = (uint16_t)f; ctrl[i] = c;
            for (int k = 0; k < 8; ++k) slots[(uint64_t)k * n + i] = s[k];
        }
    });
}
void mir_encode_batch(void* h, const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl, uint64_t n, uint32_t* words, int threads) {
    const Mirror* m = (const Mirror*)h;
    pfor(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint32_t s[8];
            for (int k = 0; k < 8; ++k) s[k] = slots[(uint64_t)k * n + i];
            encode_record<HotPlain, HotPlain>(m->view, form[i], s, ctrl[i], &words[4 * i], &words[4 * i + 1], &words[4 * i + 2], &words[4 * i + 3]);
        }
    });
}
void mir_roundtrip_batch(void* h, const uint32_t* words, uint64_t n, uint8_t* status, int threads) {
    const Mirror* m = (const Mirror*)h;
    pfor(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i)
            status[i] = (uint8_t)roundtrip_word<HotPlain>(m->view, words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3]);
    });
}
void mir_roundtrip_unfused_batch(void* h, const uint32_t* words, uint64_t n, uint8_t* status, int threads) {
    const Mirror* m = (const Mirror*)h;
    pfor(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i)
            status[i] = (uint8_t)roundtrip_word_unfused<HotPlain>(m->view, words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3]);
    });
}
void mir_synth_batch(void* h, uint32_t mix, uint64_t seed, uint32_t noise_ppm, uint64_t first, uint64_t n, uint32_t* words,
                     uint16_t* form, uint32_t* slots, uint32_t* ctrl, int threads) {
    const Mirror* m = (const Mirror*)h;
    SynthTables st = build_synth_tables(m->table, mix, seed);
    SynthView g{st.cdf.data(), st.rank_first.data(), st.rank_count.data(), (uint32_t)st.cdf.size(), noise_ppm, seed};
    pfor(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint32_t f = FORM_NONE, c = 0, s[8] = {0}, w[4];
            if (synth_record(m->view, g, first + i, &f, s, &c, w)) encode_record<HotPlain, HotPlain>(m->view, f, s, c, &w[0], &w[1], &w[2], &w[3]);
            else c = ctrl_from_raw(w[0], w[3]);
            memcpy(words + 4 * i, w, 16);
            if (form) form[i] = (uint16_t)f;
            if (ctrl) ctrl[i] = c;
            if (slots) for (int k = 0; k < 8; ++k) slots[(uint64_t)k * n + i] = s[k];
        }
    });
}
}
