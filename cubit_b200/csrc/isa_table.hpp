// ISA table: JSON -> canonical list of encoding variants.
//
// Mirrors what the reference's loader accepts and rejects (reference src/table.rs:230-434):
// unified format ("_meta" + "instructions") or the legacy flat map, hex and_base /
// variable_mask, fields validated to lie inside the 128-bit word, unknown extraction
// spellings are errors, a missing variable_mask is the OR of the field ranges, and the
// per-key ctrl_class string resolves to an epoch upper32 through _meta.ctrl_classes and
// _meta.ctrl_epochs.
//
// The reference keeps keys and modifier groups in hash maps, so its iteration order is
// random per process.  Here every (key, mod_group) pair gets a stable "variant id": its
// index when pairs are sorted bytewise by key, then by mod_group.  That id is the `form`
// value of a decoded record.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace cubit {

typedef unsigned __int128 u128;

// Extraction kinds (reference src/table.rs:52-82).  `param`/`param2` carry the numeric
// arguments of the parameterised kinds (RegShr(n), SubRShr(n, s), ...).
enum class Ext : uint8_t {
    Guard, GuardLo3, GuardNeg,
    Reg, UReg, URegFf, RegFf, Pred, Barrier,
    Imm, ImmShr, ImmDec, ImmDecU32,
    F32, F16, F16d, F64hi,
    Neg, NegShl1, Reuse, Inv, Abs, NegAbs,
    ByteSel,
    SysReg, SysRegLo7, SysRegLo4, SysRegHi4, SysRegHi1,
    RegShr, URegShr,
    SubR, SubUR, SubImm, SubImmS24,
    SubRShr, SubURShr, SubImmShr,
    Cm16Off, Cm17Off,
    OpaqueModifier,
    None,
};

struct IsaField {
    uint32_t shift = 0;
    uint32_t bits = 0;
    uint64_t mask = 0;       // (1 << bits) - 1, all ones for bits >= 64
    int32_t token_idx = 0;
    Ext ext = Ext::None;
    uint8_t param = 0, param2 = 0;
    std::string ext_name;    // the spelling a decoded field reports (reference src/decoder.rs:679-705)
    u128 range() const {
        return bits >= 128 ? ~(u128)0 : ((((u128)1 << bits) - 1) << shift);
    }
};

enum CtrlKind : uint8_t { CTRL_NORMAL = 0, CTRL_NOP = 1, CTRL_STATIC = 2 };

struct IsaVariant {
    uint32_t key_id = 0;
    std::string mod_group;
    u128 and_base = 0;
    u128 variable_mask = 0;
    std::vector<IsaField> fields;
};

struct IsaKey {
    std::string name;
    bool has_ctrl_class = false;
    std::string ctrl_class;        // raw string from the table
    CtrlKind ctrl_kind = CTRL_NORMAL;
    bool has_epoch = false;
    uint32_t epoch_upper32 = 0;
    uint32_t first_variant = 0;    // variants of one key are contiguous in canonical order
    uint32_t n_variants = 0;
};

struct IsaTable {
    std::vector<IsaKey> keys;          // bytewise sorted by name
    std::vector<IsaVariant> variants;  // canonical order

    // Throws std::runtime_error with a message naming the offending key / field.
    static IsaTable from_json_text(const std::string& text);
    static IsaTable from_file(const std::string& path);

    size_t num_keys() const { return keys.size(); }
    size_t num_groups() const { return variants.size(); }
    const std::string& key_of(uint32_t variant) const { return keys[variants[variant].key_id].name; }
};

// "0x..." (prefix optional) -> u128; more than 128 significant bits is an error.
u128 parse_hex_u128(const std::string& s);
std::string hex_u128(u128 v);

}  // namespace cubit
