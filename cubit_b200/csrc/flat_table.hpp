// Compiles the nested ISA table into the flat arrays the kernels read, plus the static
// per-variant metadata a host needs to turn a record back into named fields.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "codec_core.cuh"
#include "isa_table.hpp"

namespace cubit {

struct FieldMeta {
    uint32_t shift, bits;
    int32_t token_idx;
    uint32_t dst_pos;        // bit position of the value inside the 256-bit slot area; 0xFFFFFFFF: not stored
    uint32_t stored_bits;    // bits of the field below bit 96 of the word (what a record can hold)
    std::string name;        // Rd/Ra/Rb/Rc/guard or "[hi:lo]" (reference src/decoder.rs:668-677)
    std::string extraction;  // reference src/decoder.rs:679-705
};

struct VariantMeta {
    std::string key, mod_group, opcode;
    uint32_t key_id = 0;
    uint32_t layout_kind = 0;   // 0: one slot per multi-bit field, 1-bit fields in slot 7; 1: bits in place
    uint32_t synth_mask = 0;    // bit0: 63 (neg Rb) bit1: 62 (abs Rb) bit2: 72 (neg Ra) bit3: 73 (abs Ra)
    int32_t ra_tok = 0, rb_tok = 0;
    int32_t score = 0;
    std::vector<FieldMeta> fields;
};

struct FlatTable {
    std::vector<uint32_t> blob;      // every table, hot sections first; offsets in `at`
    BlobLayout at{};
    // Sections as built (kept for inspection; the kernels read the blob).
    std::vector<uint32_t> nodes;     // NR_WORDS each
    std::vector<uint32_t> children;  // refs
    std::vector<uint32_t> classes;   // CR_WORDS each
    std::vector<uint32_t> flagbest;  // FB_WORDS per class, indexed by the class; filled for classes that have several members
    std::vector<uint32_t> leafbest;  // FB_WORDS per class index, filled at the first class of every leaf of at most 16 classes
    std::vector<uint32_t> broad;     // BR_WORDS each
    std::vector<uint32_t> ext;       // XR_WORDS per distinct field layout
    std::vector<uint32_t> enc;       // ER_WORDS per distinct field layout: the encoder's view of `ext`
    std::vector<uint32_t> var;       // VR_WORDS per variant
    std::vector<uint32_t> gfields;
    std::vector<uint32_t> gindex;    // per variant: first generator field | count << 24
    std::vector<uint32_t> metaf;     // MF_WORDS per variant
    std::vector<uint32_t> rt;        // 4 per variant: roundtrip constants {A0, A1, A2, E3 | mask index << 9}
    std::vector<uint32_t> rt_masks;  // 4 per distinct mask: {~M0, ~M1, ~M2, reuse keep | const << 3}
    std::vector<VariantMeta> meta;
    uint32_t n_keys = 0;
    uint32_t n_buckets = 0;
    uint32_t max_bucket = 0;         // variants sharing one value of the opcode bits
    uint32_t n_leaves = 0;
    uint32_t max_leaf_classes = 0;
    uint32_t max_depth = 0;

    // Throws std::runtime_error when the table does not fit the flat encoding
    // (more than 65,534 variants, a leaf above 255 classes, a class above 255 members).
    static FlatTable compile(const IsaTable& t);
};

// Stream generator tables (which key each rank draws) for the three synthetic mixes.
enum SynthMix : uint32_t { MIX_UNIFORM = 0, MIX_ZIPF = 1, MIX_FAMILY = 2 };
struct SynthTables {
    std::vector<uint64_t> cdf;
    std::vector<uint32_t> rank_first, rank_count;
};
SynthTables build_synth_tables(const IsaTable& t, uint32_t mix, uint64_t seed);

}  // namespace cubit
