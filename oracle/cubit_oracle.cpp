// CPU ORACLE — TEST INFRASTRUCTURE, NOT PART OF THE PRODUCT.
//
// A plain C++ restatement of the SM120 codec path of kacper-daftcode/cubit, written from the
// reference's Rust sources (cited per function, paths relative to the reference repository).
// It works on the *nested* table (key -> modifier group -> entry) with strings and a real
// stable sort, the way the reference does, so that it shares no table-compilation logic
// with the GPU library it checks.  Only tests, the smoke check and the CPU-baseline leg of
// the benchmark may load it; the product library never does.
//
// Pinning: the reference is a Rust crate and no Rust toolchain exists on the build or GPU
// machines, so this oracle cannot be compared with the reference binary.  It is pinned
// instead against every golden word the reference's own tests hold for this path
// (tests/encoding.rs), see tests/golden/ and tests/test_oracle_golden.py.
//
// Two deliberate, documented departures from the reference's run-to-run behaviour:
//  * The reference iterates hash maps, so candidates that tie on the whole sort tuple come
//    out in a random order.  Here entries are visited in bytewise (key, mod_group) order, and
//    each decoded word reports `tie` when that order decided the result.
//  * The reference has no record-level encoder (its encoder takes parsed text).  The record
//    encoder here is the table-driven core of src/encoder.rs, listed at orc_encode_record.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#include "../cubit_b200/csrc/json.hpp"   // JSON text -> tree only; no codec logic lives there

typedef unsigned __int128 u128;
using cubit_json::Value;

namespace {

// ---------------------------------------------------------------------------------------
// Table (reference src/table.rs)
// ---------------------------------------------------------------------------------------

enum class X {  // extraction kinds, src/table.rs:52-82
    Guard, GuardLo3, GuardNeg, Reg, UReg, URegFf, RegFf, Pred, Barrier, Imm, ImmShr, ImmDec, ImmDecU32,
    F32, F16, F16d, F64hi, Neg, NegShl1, Reuse, Inv, Abs, NegAbs, ByteSel, SysReg, SysRegLo7, SysRegLo4,
    SysRegHi4, SysRegHi1, RegShr, URegShr, SubR, SubUR, SubImm, SubImmS24, SubRShr, SubURShr, SubImmShr,
    Cm16Off, Cm17Off, OpaqueModifier, None
};

struct Field {
    uint32_t shift, bits;
    uint64_t mask;
    int32_t token_idx;
    X ext;
    int p1 = 0, p2 = 0;
};

struct Entry {
    u128 and_base = 0, variable_mask = 0;
    std::vector<Field> fields;
};

struct KeyEntry {
    std::map<std::string, Entry> mod_groups;
    bool has_class = false;
    std::string ctrl_class;
    bool has_epoch = false;
    uint32_t epoch = 0;
};

bool starts_with(const std::string& s, const std::string& p) { return s.compare(0, p.size(), p) == 0; }
bool ends_with(const std::string& s, const std::string& p) {
    return s.size() >= p.size() && s.compare(s.size() - p.size(), p.size(), p) == 0;
}
bool contains(const std::string& s, const std::string& p) { return s.find(p) != std::string::npos; }
std::vector<std::string> split(const std::string& s, char c) {
    std::vector<std::string> out;
    std::string cur;
    for (char ch : s) {
        if (ch == c) { out.push_back(cur); cur.clear(); } else cur.push_back(ch);
    }
    out.push_back(cur);
    return out;
}
std::string trim(std::string s) {
    while (!s.empty() && isspace((unsigned char)s.back())) s.pop_back();
    size_t a = 0;
    while (a < s.size() && isspace((unsigned char)s[a])) ++a;
    return s.substr(a);
}

// src/table.rs:230-234
u128 parse_hex(const std::string& raw) {
    std::string s = trim(raw);
    if (starts_with(s, "0x") || starts_with(s, "0X")) s = s.substr(2);
    if (s.empty()) throw std::runtime_error("invalid hex: " + raw);
    u128 v = 0;
    for (char c : s) {
        int d = (c >= '0' && c <= '9') ? c - '0' : (c >= 'a' && c <= 'f') ? c - 'a' + 10 : (c >= 'A' && c <= 'F') ? c - 'A' + 10 : -1;
        if (d < 0) throw std::runtime_error("invalid hex: " + raw);
        if (v >> 124) throw std::runtime_error("invalid hex: " + raw);
        v = (v << 4) | (unsigned)d;
    }
    return v;
}

int parse_small(const std::string& s) {
    if (s.empty()) throw std::runtime_error("bad number in extraction");
    int v = 0;
    for (char c : s) {
        if (c < '0' || c > '9') throw std::runtime_error("bad number in extraction");
        v = v * 10 + (c - '0');
        if (v > 255) throw std::runtime_error("bad number in extraction");
    }
    return v;
}

// src/table.rs:84-183
void parse_extraction(const std::string& s, Field* f) {
    static const std::map<std::string, std::tuple<X, int>> fixed = {
        {"guard", {X::Guard, 0}}, {"guard_lo3", {X::GuardLo3, 0}}, {"guard_neg", {X::GuardNeg, 0}}, {"reg", {X::Reg, 0}},
        {"ureg", {X::UReg, 0}}, {"ureg_ff", {X::URegFf, 0}}, {"reg_ff", {X::RegFf, 0}}, {"pred", {X::Pred, 0}},
        {"upred", {X::Pred, 0}}, {"barrier", {X::Barrier, 0}}, {"imm", {X::Imm, 0}}, {"imm_dec", {X::ImmDec, 0}},
        {"imm_dec_u32", {X::ImmDecU32, 0}}, {"f32", {X::F32, 0}}, {"f16", {X::F16, 0}}, {"f16_d", {X::F16d, 0}},
        {"f64hi", {X::F64hi, 0}}, {"neg", {X::Neg, 0}}, {"neg_shl1", {X::NegShl1, 0}}, {"reuse", {X::Reuse, 0}},
        {"inv", {X::Inv, 0}}, {"abs", {X::Abs, 0}}, {"neg_abs", {X::NegAbs, 0}}, {"byte_sel", {X::ByteSel, 0}},
        {"sysreg", {X::SysReg, 0}}, {"sysreg_lo7", {X::SysRegLo7, 0}}, {"sysreg_lo4", {X::SysRegLo4, 0}},
        {"sysreg_hi4", {X::SysRegHi4, 0}}, {"sysreg_hi1", {X::SysRegHi1, 0}}, {"sub_r0", {X::SubR, 0}},
        {"sub_r1", {X::SubR, 1}}, {"sub_r2", {X::SubR, 2}}, {"sub_ur0", {X::SubUR, 0}}, {"sub_ur1", {X::SubUR, 1}},
        {"sub_imm0", {X::SubImm, 0}}, {"sub_imm1", {X::SubImm, 1}}, {"sub_imm2", {X::SubImm, 2}},
        {"sub_imm0_s24", {X::SubImmS24, 0}}, {"sub_imm1_s24", {X::SubImmS24, 1}}, {"sub_imm2_s24", {X::SubImmS24, 2}},
        {"cm16_off", {X::Cm16Off, 0}}, {"cm17_off", {X::Cm17Off, 0}}, {"opaque_mod", {X::OpaqueModifier, 0}},
        {"", {X::None, 0}},
    };
    auto it = fixed.find(s);
    if (it != fixed.end()) { f->ext = std::get<0>(it->second); f->p1 = std::get<1>(it->second); return; }
    if (starts_with(s, "reg_shr")) { f->ext = X::RegShr; f->p1 = parse_small(s.substr(7)); return; }
    if (starts_with(s, "ureg_shr")) { f->ext = X::URegShr; f->p1 = parse_small(s.substr(8)); return; }
    if (starts_with(s, "imm_shr")) { f->ext = X::ImmShr; f->p1 = parse_small(s.substr(7)); return; }
    struct { const char* prefix; const char* tag; X kind; } subs[] = {
        {"sub_r", "r", X::SubRShr}, {"sub_ur", "ur", X::SubURShr}, {"sub_imm", "imm", X::SubImmShr}};
    for (auto& sb : subs) {
        if (starts_with(s, sb.prefix) && contains(s, "_shr")) {
            std::vector<std::string> parts = split(s, '_');
            if (parts.size() < 3 || !starts_with(parts[1], sb.tag) || !starts_with(parts[2], "shr"))
                throw std::runtime_error("invalid extraction '" + s + "'");
            f->ext = sb.kind;
            f->p1 = parse_small(parts[1].substr(strlen(sb.tag)));
            f->p2 = parse_small(parts[2].substr(3));
            return;
        }
    }
    throw std::runtime_error("unknown extraction '" + s + "'");
}

// Spelling a decoded field reports, src/decoder.rs:679-705 (the catch-all arm is the
// lower-cased Rust Debug name of the variant).
std::string extraction_name(const Field& f) {
    switch (f.ext) {
        case X::Guard: return "guard"; case X::Reg: return "reg"; case X::UReg: return "ureg";
        case X::URegFf: return "ureg_ff"; case X::RegFf: return "reg_ff";
        case X::RegShr: return "reg_shr" + std::to_string(f.p1);
        case X::URegShr: return "ureg_shr" + std::to_string(f.p1);
        case X::Pred: return "pred"; case X::Imm: return "imm";
        case X::ImmShr: return "imm_shr" + std::to_string(f.p1);
        case X::Reuse: return "reuse"; case X::Neg: return "neg"; case X::F32: return "f32"; case X::F16d: return "f16_d";
        case X::SubR: return "sub_r" + std::to_string(f.p1);
        case X::SubUR: return "sub_ur" + std::to_string(f.p1);
        case X::SubImm: return "sub_imm" + std::to_string(f.p1);
        case X::SubRShr: return "sub_r" + std::to_string(f.p1) + "_shr" + std::to_string(f.p2);
        case X::SubURShr: return "sub_ur" + std::to_string(f.p1) + "_shr" + std::to_string(f.p2);
        case X::SubImmShr: return "sub_imm" + std::to_string(f.p1) + "_shr" + std::to_string(f.p2);
        case X::SubImmS24: return "sub_imm" + std::to_string(f.p1) + "_s24";
        case X::OpaqueModifier: return "opaque_mod";
        case X::GuardLo3: return "guardlo3"; case X::GuardNeg: return "guardneg"; case X::Barrier: return "barrier";
        case X::ImmDec: return "immdec"; case X::ImmDecU32: return "immdecu32"; case X::F16: return "f16";
        case X::F64hi: return "f64hi"; case X::NegShl1: return "negshl1"; case X::Inv: return "inv";
        case X::Abs: return "abs"; case X::NegAbs: return "negabs"; case X::ByteSel: return "bytesel";
        case X::SysReg: return "sysreg"; case X::SysRegLo7: return "sysreglo7"; case X::SysRegLo4: return "sysreglo4";
        case X::SysRegHi4: return "sysreghi4"; case X::SysRegHi1: return "sysreghi1";
        case X::Cm16Off: return "cm16off"; case X::Cm17Off: return "cm17off"; case X::None: return "none";
    }
    return "none";
}

u128 field_range(const Field& f) { return f.bits >= 128 ? ~(u128)0 : ((((u128)1 << f.bits) - 1) << f.shift); }

struct Table {
    std::map<std::string, KeyEntry> entries;   // bytewise order = canonical order

    const Entry* get(const std::string& key, const std::string& mg) const {   // src/table.rs:406-408
        auto it = entries.find(key);
        if (it == entries.end()) return nullptr;
        auto jt = it->second.mod_groups.find(mg);
        return jt == it->second.mod_groups.end() ? nullptr : &jt->second;
    }
};

uint32_t want_u32(const Value* v, const std::string& where) {
    if (!v || v->kind != Value::Number || !v->is_integer || v->is_negative || v->mag > 0xFFFFFFFFull)
        throw std::runtime_error("failed to parse table JSON (" + where + ")");
    return (uint32_t)v->mag;
}

// src/table.rs:346-403
void parse_groups(const std::string& key, const Value& groups, KeyEntry* ke) {
    if (!groups.is_object()) throw std::runtime_error("failed to parse table JSON (mod_groups of " + key + ")");
    for (const auto& m : groups.obj) {
        const std::string& mods = m.first;
        const Value& g = m.second;
        const std::string where = key + "::" + mods;
        const Value* ab = g.get("and_base");
        const Value* fl = g.get("fields");
        if (!ab || !ab->is_string() || !fl || !fl->is_array()) throw std::runtime_error("failed to parse table JSON (" + where + ")");
        Entry e;
        e.and_base = parse_hex(ab->str);
        for (const Value& jf : fl->arr) {
            Field f;
            f.shift = want_u32(jf.get("shift"), where);
            f.bits = want_u32(jf.get("bits"), where);
            const Value* tk = jf.get("token_idx");
            if (!tk || tk->kind != Value::Number || !tk->is_integer || tk->mag > 0x80000000ull)
                throw std::runtime_error("failed to parse table JSON (" + where + ")");
            f.token_idx = tk->is_negative ? (int32_t)(-(int64_t)tk->mag) : (int32_t)tk->mag;
            const Value* ex = jf.get("extraction");
            if (!ex || !ex->is_string()) throw std::runtime_error("failed to parse table JSON (" + where + ")");
            if (f.bits == 0 || (uint64_t)f.shift + f.bits > 128)
                throw std::runtime_error("field outside 128-bit instruction for " + where);
            f.mask = f.bits >= 64 ? ~0ull : ((1ull << f.bits) - 1);
            parse_extraction(ex->str, &f);
            e.fields.push_back(f);
        }
        const Value* vm = g.get("variable_mask");
        if (vm && vm->kind != Value::Null) {
            if (!vm->is_string()) throw std::runtime_error("failed to parse table JSON (" + where + ")");
            e.variable_mask = parse_hex(vm->str);
        } else {
            for (const Field& f : e.fields) e.variable_mask |= field_range(f);
        }
        ke->mod_groups[mods] = e;   // a repeated name keeps the last entry
    }
}

// src/table.rs:251-343
Table load_table(const std::string& text) {
    Value root = cubit_json::parse(text);
    Table t;
    const bool unified = contains(text, "\"_meta\"") && contains(text, "\"instructions\"");
    if (!unified) {
        for (const auto& m : root.obj) {
            const Value* groups = m.second.get("mod_groups");
            if (!groups) throw std::runtime_error("failed to parse table JSON (missing mod_groups)");
            KeyEntry ke;
            parse_groups(m.first, *groups, &ke);
            t.entries[m.first] = ke;
        }
        return t;
    }
    std::map<std::string, uint32_t> epochs, class_epoch;
    if (const Value* meta = root.get("_meta")) {
        if (const Value* ce = meta->get("ctrl_epochs"))
            for (const auto& m : ce->obj) {
                const Value* up = m.second.get("upper32");
                if (up && up->is_string()) {
                    try { epochs[m.first] = (uint32_t)parse_hex(up->str); } catch (...) {}
                }
            }
        if (const Value* cc = meta->get("ctrl_classes"))
            for (const auto& m : cc->obj) {
                const Value* en = m.second.get("hi_upper32");
                if (en && en->is_string() && epochs.count(en->str)) class_epoch[m.first] = epochs[en->str];
            }
    }
    const Value* ins = root.get("instructions");
    if (!ins || !ins->is_object()) throw std::runtime_error("missing 'instructions' key");
    for (const auto& m : ins->obj) {
        const Value* groups = m.second.get("mod_groups");
        if (!groups) continue;
        KeyEntry ke;
        parse_groups(m.first, *groups, &ke);
        const Value* cc = m.second.get("ctrl_class");
        if (cc && cc->is_string()) {
            ke.has_class = true;
            ke.ctrl_class = cc->str;
            auto it = class_epoch.find(cc->str);
            if (it != class_epoch.end()) { ke.has_epoch = true; ke.epoch = it->second; }
        }
        t.entries[m.first] = ke;
    }
    return t;
}

// ---------------------------------------------------------------------------------------
// Decoder (reference src/decoder.rs)
// ---------------------------------------------------------------------------------------

const char* const OP_TYPES[] = {"ARURR", "ARURI", "ARUR", "AURI", "AURR", "AUR", "cAI", "dARI", "ARI", "UP", "UR",
                                "SR", "FI", "II", "IM", "LO", "R", "P", "L", "B", "?"};   // :602-607
bool in_op_types(const std::string& s) {
    for (const char* t : OP_TYPES)
        if (s == t) return true;
    return false;
}

// :609-618
std::vector<std::string> parse_ins_key_op_types(const std::string& key) {
    std::vector<std::string> out;
    bool in_ops = false;
    for (const std::string& part : split(key, '_')) {
        if (!in_ops && in_op_types(part)) in_ops = true;
        if (in_ops) out.push_back(part);
    }
    return out;
}

// :623-666
int key_field_consistency_score(const std::string& key, const std::string& mg, const Table& table) {
    const Entry* entry = table.get(key, mg);
    if (!entry) return 0;
    std::vector<std::string> op_types = parse_ins_key_op_types(key);
    int score = 0;
    for (const Field& f : entry->fields) {
        if (f.token_idx <= 0) continue;
        size_t idx = (size_t)(f.token_idx - 1);
        std::string op_type = idx < op_types.size() ? op_types[idx] : "";
        std::string ext = extraction_name(f);
        bool is_pred = ext == "pred" || ext == "guard";
        bool is_upred = ext == "upred";
        bool is_reg = ext == "reg" || ext == "ureg" || ext == "ureg_ff" || ext == "reg_ff" || ext == "reg_shr1" ||
                      ext == "reg_shr2" || ext == "reg_shr3";
        bool is_imm = starts_with(ext, "imm") || ext == "f32" || ext == "f16" || ext == "f16_d" || ext == "f64hi";
        bool is_barrier = ext == "barrier";
        bool e_pred = op_type == "P", e_upred = op_type == "UP", e_reg = op_type == "R" || op_type == "UR";
        bool e_imm = op_type == "II" || op_type == "IM" || op_type == "LO" || op_type == "FI", e_bar = op_type == "B";
        if (e_pred && is_pred) score += 2;
        else if (e_upred && is_upred) score += 4;
        else if (e_bar && is_barrier) score += 4;
        else if ((e_upred && is_pred) || (e_pred && is_upred)) score -= 2;
        else if ((e_reg && is_reg) || (e_imm && is_imm)) score += 2;
        else if ((e_pred && is_reg) || (e_reg && is_pred)) score -= 5;
        else if (e_reg && is_imm) score -= 4;
        else if (e_imm && is_reg) score -= 2;
        else if (e_bar && is_pred) score -= 5;
        bool is_subur = starts_with(ext, "sub_ur");
        bool e_desc = op_type == "dARI" || op_type == "ARURI";
        if (e_desc && is_subur) score += 3;
    }
    return score;
}

// :581-599
bool key_has_output_pred_field(const std::string& key, const std::string& mg, const Table& table) {
    std::vector<std::string> op_types = parse_ins_key_op_types(key);
    for (size_t i = 1; i < op_types.size(); ++i)
        if (op_types[i] == "P" || op_types[i] == "UP") return true;
    if (const Entry* e = table.get(key, mg))
        for (const Field& f : e->fields)
            if (f.token_idx >= 1 && f.ext == X::Pred) return true;
    return false;
}

bool has_middle_pred(const std::string& key) {   // :491-494, :556-559
    std::vector<std::string> t = parse_ins_key_op_types(key);
    if (t.size() <= 2) return false;
    for (size_t i = 1; i + 1 < t.size(); ++i)
        if (t[i] == "P" || t[i] == "UP") return true;
    return false;
}

struct Candidate {   // :67-76
    std::string key, mod_group;
    u128 and_base, match_mask, relaxed_match_mask, broad_relaxed_match_mask;
    uint32_t variant;   // canonical id (not in the reference)
    // Static sort components, cached at build time; each is computed by the literal function.
    int score, opaque_penalty, plain_addr_penalty, undiscovered_penalty, key_len, match_popcount, mg_len;
    bool no_fields, is_mem_addr;
};

int popcount128(u128 v) { return __builtin_popcountll((uint64_t)v) + __builtin_popcountll((uint64_t)(v >> 64)); }

struct DecodeIndex {
    std::map<uint16_t, std::vector<Candidate>> opcode_map;

    // :80-160, plus the per-candidate parts of the sort key at :213-279
    void build(const Table& table) {
        uint32_t variant = 0;
        for (const auto& kv : table.entries) {
            const std::string& key = kv.first;
            for (const auto& gv : kv.second.mod_groups) {
                const Entry& mg = gv.second;
                Candidate c;
                c.key = key; c.mod_group = gv.first; c.and_base = mg.and_base; c.variant = variant++;
                u128 field_mask = 0, imm_extra = 0;
                for (const Field& f : mg.fields) {
                    field_mask |= field_range(f);
                    switch (f.ext) {
                        case X::Imm: case X::ImmShr: case X::ImmDec: case X::ImmDecU32: case X::F32: case X::F16: case X::F16d:
                        case X::F64hi: case X::SubR: case X::SubUR: case X::SubImm: case X::SubImmS24: case X::SubRShr:
                        case X::SubURShr: case X::SubImmShr: imm_extra |= field_range(f); break;
                        default: break;
                    }
                }
                c.match_mask = ~mg.variable_mask & ~field_mask;
                c.relaxed_match_mask = c.match_mask & ~imm_extra;
                const u128 std_reg = ((u128)0xFF << 16) | ((u128)0xFF << 24) | ((u128)0xFFFFFFFFull << 32) | ((u128)0xFF << 64);
                c.broad_relaxed_match_mask = c.relaxed_match_mask & ~std_reg;
                c.no_fields = mg.fields.empty();
                c.is_mem_addr = contains(key, "_ARI") || contains(key, "_AI") || contains(key, "dARI") || contains(key, "ARURI");
                c.score = key_field_consistency_score(key, gv.first, table);
                c.opaque_penalty = 0;
                for (const Field& f : mg.fields)
                    if (f.ext == X::OpaqueModifier) c.opaque_penalty = 1;
                bool is_global = starts_with(key, "LDG") || starts_with(key, "STG") || starts_with(key, "LDGSTS") ||
                                 starts_with(key, "ATOMG") || starts_with(key, "REDG");
                if (!is_global || contains(key, "dARI") || contains(key, "dAI")) c.plain_addr_penalty = 0;
                else if (contains(key, "_ARI") || contains(key, "_AI")) c.plain_addr_penalty = 1;
                else c.plain_addr_penalty = 0;
                bool undiscovered = ends_with(key, "_?") || contains(key, "_?_") || contains(key, "_II_?");
                bool excess = contains(key, "_II_II_UR") || contains(key, "_II_UR") || contains(key, "_UR_II") ||
                              contains(key, "_II_II_?") || contains(key, "_R_II_?") || contains(key, "_P_II_II");
                c.undiscovered_penalty = undiscovered ? 50 : (excess ? 30 : 0);
                c.key_len = (int)key.size();
                c.match_popcount = popcount128(c.match_mask);
                c.mg_len = (int)gv.first.size();
                opcode_map[(uint16_t)(mg.and_base & 0x0FFF)].push_back(c);
            }
        }
    }
};

struct Match {
    const Candidate* c;
    int priority;
    std::tuple<int, int, int, int, int, int, int, int, int, int> sort_key;
};

bool explicit_mode(const Candidate& c, const std::string& m) {   // :408-411
    std::vector<std::string> dotted = split(split(c.key, '_')[0], '.');
    for (size_t i = 1; i < dotted.size(); ++i)
        if (dotted[i] == m) return true;
    return false;
}
bool grouped_mode(const Candidate& c, const std::string& m) {   // :412-414
    for (const std::string& x : split(c.mod_group, ','))
        if (trim(x) == m) return true;
    return false;
}
bool has_pred_field(const Table& t, const Candidate& c, uint32_t min_shift) {
    const Entry* e = t.get(c.key, c.mod_group);
    if (!e) return false;
    for (const Field& f : e->fields)
        if (f.shift >= min_shift && f.ext == X::Pred) return true;
    return false;
}
bool has_early_output_pred(const Table& t, const Candidate& c) {   // :538-542
    const Entry* e = t.get(c.key, c.mod_group);
    if (!e) return false;
    for (const Field& f : e->fields)
        if (f.token_idx >= 1 && f.token_idx <= 3 && f.ext == X::Pred && f.shift >= 80 && f.shift <= 85) return true;
    return false;
}

// :391-574.  Returns the index into `matches`, or -1.  `tie` reports whether the choice
// rests on the order of candidates whose whole sort tuple is equal.
int select_best_candidate(const std::vector<Match>& matches, u128 cc, const Table& table, bool* tie) {
    *tie = false;
    if (matches.empty()) return -1;
    const Candidate& first = *matches[0].c;
    const bool tie_first = matches.size() > 1 && matches[1].sort_key == matches[0].sort_key;
    // Picks the first candidate satisfying `pred`; the tie flag then also covers other
    // satisfying candidates with the same tuple.
    auto pick = [&](auto pred) -> int {
        for (size_t i = 0; i < matches.size(); ++i)
            if (pred(*matches[i].c)) {
                bool t = tie_first;
                if (i != 0)
                    for (size_t j = 0; j < matches.size(); ++j)
                        if (j != i && matches[j].sort_key == matches[i].sort_key && pred(*matches[j].c)) t = true;
                *tie = t;
                return (int)i;
            }
        return -1;
    };
    int r;
    bool any_bra = false;
    for (const Match& m : matches) any_bra |= starts_with(m.c->key, "BRA");
    if (any_bra) {   // :401-431
        const char* mode = nullptr;
        switch ((unsigned)((cc >> 32) & 3)) { case 1: mode = "U"; break; case 2: mode = "DIV"; break; case 3: mode = "CONV"; break; default: break; }
        if (mode) {
            if ((r = pick([&](const Candidate& c) { return explicit_mode(c, mode); })) >= 0) return r;
            if ((r = pick([&](const Candidate& c) { return grouped_mode(c, mode); })) >= 0) return r;
        } else {
            r = pick([&](const Candidate& c) {
                for (const char* m : {"U", "DIV", "CONV"})
                    if (explicit_mode(c, m) || grouped_mode(c, m)) return false;
                return true;
            });
            if (r >= 0) return r;
        }
    }
    if (const Entry* e = table.get(first.key, first.mod_group)) {   // :437-459
        for (const Field& f : e->fields) {
            if (f.token_idx >= 1 && f.token_idx <= 3 && f.shift >= 80 && f.shift <= 85 && f.ext == X::Pred) {
                uint64_t mask = (1ull << f.bits) - 1;
                uint64_t val = (uint64_t)(cc >> f.shift) & mask;
                if (val == mask) {
                    r = pick([&](const Candidate& c) { return !key_has_output_pred_field(c.key, c.mod_group, table); });
                    if (r >= 0) return r;
                }
                break;
            }
        }
    }
    if (((cc >> 64) & 0xff) == 0xff) {   // :465-473
        r = pick([&](const Candidate& c) { return c.score >= 0 && contains(c.mod_group, "SHL"); });
        if (r >= 0) return r;
    }
    const unsigned trailing = (unsigned)((cc >> 87) & 0xF);   // :478-515
    if (trailing != 0x7 && trailing != 0xF) {
        if (starts_with(first.key, "LEA_") || starts_with(first.key, "ULEA_")) {
            const bool output_is_pt = ((cc >> 81) & 7) == 7;
            r = pick([&](const Candidate& c) {
                if (!(ends_with(c.key, "_P") || ends_with(c.key, "_UP"))) return false;
                if (output_is_pt && has_middle_pred(c.key)) return false;
                return has_pred_field(table, c, 87);
            });
            if (r >= 0) return r;
        }
        r = pick([&](const Candidate& c) { return has_pred_field(table, c, 87); });
        if (r >= 0) return r;
    }
    if (starts_with(first.key, "ULOP3") || starts_with(first.key, "UPLOP3")) {   // :520-526
        r = pick([&](const Candidate& c) { return ends_with(c.key, "_UP"); });
        if (r >= 0) return r;
    }
    const unsigned out_pred = (unsigned)((cc >> 81) & 7);   // :534-571
    if (out_pred != 7) {
        r = pick([&](const Candidate& c) { return has_early_output_pred(table, c); });
        if (r >= 0) return r;
    }
    if (out_pred == 7 && has_middle_pred(first.key)) {
        r = pick([&](const Candidate& c) { return !has_middle_pred(c.key); });
        if (r >= 0) return r;
    }
    *tie = tie_first;
    return 0;
}

struct Decoded {
    int status;          // 0 ok, 1 no opcode bucket (:172-173), 2 no candidate matches (:286-287)
    uint32_t variant;
    const Candidate* cand;
    const Entry* entry;
    std::vector<uint64_t> values;   // table fields, table order
    unsigned synth;                 // bit0: 63, bit1: 62, bit2: 72, bit3: 73
    unsigned stall, yield, wbar, rbar, wait;
    bool tie;
};

struct Oracle {
    Table table;
    DecodeIndex index;
    std::vector<const Candidate*> by_variant;
    std::vector<std::pair<std::string, std::string>> names;
    std::map<std::pair<std::string, std::string>, uint32_t> variant_of;

    // :163-382
    Decoded decode(u128 code) const {
        Decoded d{};
        const u128 sched_mask = (u128)0xFFFFFFFFull << 96;
        const u128 cc = code & ~sched_mask;
        const unsigned ctrl_bits = (unsigned)((code >> 105) & 0x1FFFF);   // :348-355
        d.stall = ctrl_bits & 0xF; d.yield = (ctrl_bits >> 4) & 1; d.wbar = (ctrl_bits >> 5) & 7;
        d.rbar = (ctrl_bits >> 8) & 7; d.wait = (ctrl_bits >> 11) & 0x3F;
        d.variant = 0xFFFF;
        auto it = index.opcode_map.find((uint16_t)(cc & 0x0FFF));
        if (it == index.opcode_map.end()) { d.status = 1; return d; }
        const u128 guard_mask = 0xF000;
        std::vector<Match> matches;
        for (const Candidate& c : it->second) {   // :192-209
            bool strict = (cc & c.match_mask & ~guard_mask) == (c.and_base & c.match_mask & ~guard_mask);
            bool relaxed = (cc & c.relaxed_match_mask & ~guard_mask) == (c.and_base & c.relaxed_match_mask & ~guard_mask);
            int prio = -1;
            if (strict) prio = 0;
            else if (relaxed) prio = 1;
            else if (c.no_fields || c.is_mem_addr) {
                bool broad = (cc & c.broad_relaxed_match_mask & ~guard_mask) == (c.and_base & c.broad_relaxed_match_mask & ~guard_mask);
                if (broad) prio = 2;
            }
            if (prio < 0) continue;
            Match m;
            m.c = &c; m.priority = prio;
            const int bonus = c.score >= 3 ? 10 : 0;   // :246-247
            m.sort_key = std::make_tuple(c.score < 0 ? 1 : 0, prio, c.opaque_penalty, c.plain_addr_penalty,
                                         c.undiscovered_penalty, c.key_len - bonus, -c.score,
                                         -popcount128(c.and_base & cc), -c.match_popcount, -c.mg_len);   // :278
            matches.push_back(m);
        }
        std::stable_sort(matches.begin(), matches.end(), [](const Match& a, const Match& b) { return a.sort_key < b.sort_key; });
        bool tie = false;
        int sel = select_best_candidate(matches, cc, table, &tie);
        if (sel < 0) { d.status = 2; return d; }
        const Candidate& m = *matches[sel].c;
        d.status = 0; d.cand = &m; d.variant = m.variant; d.tie = tie;
        d.entry = table.get(m.key, m.mod_group);
        for (const Field& f : d.entry->fields) {   // :294-304
            uint64_t mask = f.bits >= 64 ? ~0ull : ((1ull << f.bits) - 1);
            d.values.push_back((uint64_t)(cc >> f.shift) & mask);
        }
        // :312-345
        std::string base_op = split(split(m.key, '_')[0], '.')[0];
        static const char* not_alu[] = {"LDG", "LDL", "LDS", "LDC", "LDCU", "STG", "STL", "STS", "ATOM", "RED", "BRA", "BSSY",
                                        "BSYNC", "EXIT", "RET", "BAR", "S2R", "S2UR", "LDSM", "LDGSTS", "QMMA"};
        bool is_alu = true;
        for (const char* n : not_alu) if (base_op == n) is_alu = false;
        if (is_alu) {
            const int bits[4] = {63, 62, 72, 73};
            for (int k = 0; k < 4; ++k) {
                const uint64_t bit = (uint64_t)bits[k];
                bool covered = false;
                for (const Field& f : d.entry->fields) covered |= (uint64_t)f.shift <= bit && bit < (uint64_t)f.shift + f.bits;
                bool baked = ((m.and_base >> bit) & 1) == 1;
                if (((cc >> bit) & 1) == 1 && !baked && !covered) d.synth |= 1u << k;
            }
        }
        return d;
    }
};

// Opcode text of a key, src/decoder.rs:357-371: the '_'-separated segments before the first
// operand-type segment; "B" right after a segment ending in "PACK" is a lane suffix and stays.
std::string opcode_of_key(const std::string& key) {
    std::vector<std::string> parts = split(key, '_'), op;
    for (const std::string& part : parts) {
        if (in_op_types(part)) {
            bool pack_b = part == "B" && !op.empty() && ends_with(op.back(), "PACK");
            if (!pack_b) break;
        }
        op.push_back(part);
    }
    if (op.empty()) return parts[0];
    std::string out = op[0];
    for (size_t i = 1; i < op.size(); ++i) out += "_" + op[i];
    return out;
}

// Kernel metadata from code bytes, src/main.rs:787-845: largest register number below 255,
// offsets of EXIT instructions, set of BSSY barrier indices; words that do not decode fall
// back to the fixed register byte positions and the raw opcode bits.
struct KernelMetaResult {
    uint32_t max_reg = 0, barrier_mask = 0;
    std::vector<uint32_t> exit_offsets;
};
KernelMetaResult infer_kernel_meta(const Oracle& o, const uint8_t* code, uint64_t nbytes) {
    KernelMetaResult r;
    for (uint64_t i = 0; (i + 1) * 16 <= nbytes; ++i) {
        uint64_t lo, hi;
        memcpy(&lo, code + 16 * i, 8); memcpy(&hi, code + 16 * i + 8, 8);
        const uint32_t addr = (uint32_t)(i * 16);
        Decoded d = o.decode(((u128)hi << 64) | lo);
        if (d.status == 0) {
            const std::string opcode = opcode_of_key(d.cand->key);
            for (size_t f = 0; f < d.values.size(); ++f)
                if (extraction_name(d.entry->fields[f]) == "reg") {
                    uint32_t v = (uint32_t)d.values[f];
                    if (v < 255 && v > r.max_reg) r.max_reg = v;
                }
            if (opcode == "EXIT") r.exit_offsets.push_back(addr);
            if (opcode == "BSSY")
                for (size_t f = 0; f < d.values.size(); ++f) {
                    std::string e = extraction_name(d.entry->fields[f]);
                    if ((e == "barrier" || e == "imm") && d.values[f] < 8) r.barrier_mask |= 1u << d.values[f];
                }
        } else {
            for (int shift : {16, 24, 32, 64}) {
                uint32_t v = shift < 64 ? (uint32_t)((lo >> shift) & 0xFF) : (uint32_t)(hi & 0xFF);
                if (v < 255 && v > r.max_reg) r.max_reg = v;
            }
            const uint64_t opcode = lo & 0x0FFF;
            if (opcode == 0x0918) r.exit_offsets.push_back(addr);
            if (opcode == 0x0945) r.barrier_mask |= 1u << ((lo >> 16) & 0x7);
        }
    }
    return r;
}

// ---------------------------------------------------------------------------------------
// Record layout: where the field values of a variant live in the 8 x u32 slots
// ---------------------------------------------------------------------------------------

// Only the part of a field below bit 96 is stored (the decoder never sees more).
// Layout 0: every multi-bit field has a slot of its own, handed out by the 32-bit limb of the
// word it lies in, in table order: fields of bits 31:0 take slots 0, 1, 2; of bits 63:32 slots
// 3, 5, 6; of bits 95:64 slots 4, 6, 5.  1-bit fields share slot 7 at (source bit mod 32),
// rotated left by r1 for fields in bits 63:32 and r2 for bits 95:64, (r1, r2) being the first
// pair in (0,0), (0,1), ... that keeps the three groups apart.  Layout 1, when layout 0 does
// not fit (a multi-bit field crosses a limb boundary, more than three fields in bits 31:0,
// more than two fields beyond the first of bits 63:32 and the first of bits 95:64 together,
// two 1-bit fields on one bit, no rotation) or stored field ranges overlap: every field stays
// at its position in the word.
const uint32_t NOT_STORED = 0xFFFFFFFFu;
struct Layout {
    std::vector<uint32_t> pos, stored;
    int kind;
};
uint32_t rotl32(uint32_t x, uint32_t r) { return r ? ((x << r) | (x >> (32 - r))) : x; }

Layout slot_layout(const Entry& e) {
    Layout L;
    u128 used = 0;
    bool overlap = false, dup = false, crossing = false;
    uint32_t in_limb[3] = {0, 0, 0}, fm[3] = {0, 0, 0};
    for (const Field& f : e.fields) {
        uint32_t sb = f.shift >= 96 ? 0 : std::min<uint32_t>(f.shift + f.bits, 96) - f.shift;
        L.stored.push_back(sb);
        if (!sb) continue;
        u128 r = ((((u128)1) << sb) - 1) << f.shift;
        if (used & r) overlap = true;
        used |= r;
        if (sb == 1) {
            if (fm[f.shift >> 5] >> (f.shift & 31) & 1) dup = true;
            fm[f.shift >> 5] |= 1u << (f.shift & 31);
        } else if (f.shift / 32 != (f.shift + sb - 1) / 32) crossing = true;
        else ++in_limb[f.shift / 32];
    }
    const bool flags = fm[0] | fm[1] | fm[2];
    uint32_t r1 = 0, r2 = 0;
    bool rot_ok = !flags;
    for (uint32_t a = 0; a < 32 && !rot_ok; ++a)
        for (uint32_t b = 0; b < 32 && !rot_ok; ++b) {
            uint32_t x = fm[0], y = rotl32(fm[1], a), z = rotl32(fm[2], b);
            if (!(x & y) && !(x & z) && !(y & z)) { rot_ok = true; r1 = a; r2 = b; }
        }
    const uint32_t beyond = (in_limb[1] > 1 ? in_limb[1] - 1 : 0) + (in_limb[2] > 1 ? in_limb[2] - 1 : 0);
    L.kind = (!overlap && !dup && !crossing && rot_ok && in_limb[0] <= 3 && beyond <= 2) ? 0 : 1;
    const uint32_t order[3][3] = {{0, 1, 2}, {3, 5, 6}, {4, 6, 5}};
    uint32_t next[3] = {0, 0, 0};
    for (size_t i = 0; i < e.fields.size(); ++i) {
        const Field& f = e.fields[i];
        const uint32_t sb = L.stored[i];
        if (!sb) L.pos.push_back(NOT_STORED);
        else if (L.kind == 1) L.pos.push_back(f.shift);
        else if (sb == 1) {
            const uint32_t limb = f.shift >> 5, r = limb == 0 ? 0 : (limb == 1 ? r1 : r2);
            L.pos.push_back(224 + (((f.shift & 31) + r) & 31));
        } else L.pos.push_back(32 * order[f.shift / 32][next[f.shift / 32]++]);
    }
    return L;
}

// Writes `nbits` of v at bit `pos` of the slot area, replacing what was there.
void put_bits(uint32_t slots[8], uint32_t pos, uint32_t nbits, uint64_t v) {
    for (uint32_t b = 0; b < nbits; ++b) {
        uint32_t& w = slots[(pos + b) >> 5];
        const uint32_t bit = 1u << ((pos + b) & 31);
        if ((v >> b) & 1) w |= bit; else w &= ~bit;
    }
}
uint64_t get_bits(const uint32_t slots[8], uint32_t pos, uint32_t nbits) {
    uint64_t v = 0;
    for (uint32_t b = 0; b < nbits; ++b)
        if ((slots[(pos + b) >> 5] >> ((pos + b) & 31)) & 1) v |= 1ull << b;
    return v;
}

uint32_t pack_ctrl(u128 raw, unsigned synth, bool tie, unsigned status) {
    uint32_t c = (uint32_t)((raw >> 105) & 0x1FFFF);
    c |= (uint32_t)((raw >> 122) & 7) << 17;
    c |= (uint32_t)((raw >> 12) & 0xF) << 20;
    c |= synth << 24;
    c |= (tie ? 1u : 0u) << 28;
    c |= status << 30;
    return c;
}

void decode_to_record(const Oracle& o, u128 code, uint16_t* form, uint32_t slots[8], uint32_t* ctrl) {
    Decoded d = o.decode(code);
    for (int s = 0; s < 8; ++s) slots[s] = 0;
    if (d.status != 0) { *form = 0xFFFF; *ctrl = pack_ctrl(code, 0, false, (unsigned)d.status); return; }
    Layout L = slot_layout(*d.entry);
    for (size_t i = 0; i < d.values.size(); ++i)
        if (L.pos[i] != NOT_STORED) put_bits(slots, L.pos[i], L.stored[i], d.values[i]);
    *form = (uint16_t)d.variant;
    *ctrl = pack_ctrl(code, d.synth, d.tie, 0);
}

// ---------------------------------------------------------------------------------------
// Record-level encode (the table-driven core of reference src/encoder.rs)
// ---------------------------------------------------------------------------------------

// Inputs: variant, one u64 per table field, synthesized-modifier presence, guard nibble,
// reuse3, 17-bit scheduling word.  Steps, with the reference lines they restate:
//   1. code = and_base                                                           (:293)
//   2. fields in table order, later ones overwrite earlier ones                  (:296-300)
//      A decoded record never carries field bits at or above bit 96 (the decoder reads
//      the word with bits 127:96 cleared), so those bits of a value are ignored; a `reuse`
//      field lying inside bits 124:122 takes its bits from reuse3 instead, which is what
//      the reference's text path does (printer reads the raw reuse bits, encoder feeds
//      them back through the field).
//   3. synthesized abs/neg bits 62/63/72/73 (only where decode could have produced them)  (:341-360)
//   4. guard nibble unless the entry has a full guard field                      (:368-384)
//   5. QMMA with ".SP" in the mnemonic: clear bit 80                             (:530-532)
//   6. reuse slots: bit 122+i follows reuse3[i] when the 8-bit register field at shift
//      24/32/64 has no explicit reuse field on its token                         (:1155-1179)
//   7. upper 32 bits rebuilt from reuse bits, scheduling word and the key's ctrl class  (:560-608)
u128 orc_encode_record(const Oracle& o, uint32_t variant, const std::vector<uint64_t>& values, unsigned synth,
                       unsigned guard, unsigned reuse3, unsigned sched17) {
    const Candidate& c = *o.by_variant[variant];
    const Entry& e = *o.table.get(c.key, c.mod_group);
    const KeyEntry& ke = o.table.entries.at(c.key);
    u128 code = e.and_base;
    for (size_t i = 0; i < e.fields.size(); ++i) {
        const Field& f = e.fields[i];
        uint64_t v = values[i] & f.mask;
        if (f.shift >= 96) v = 0;
        else if (f.shift + f.bits > 96 && 96 - f.shift < 64) v &= (1ull << (96 - f.shift)) - 1;
        if (f.ext == X::Reuse && f.shift >= 122 && f.shift + f.bits <= 125) v = (reuse3 >> (f.shift - 122)) & f.mask;
        u128 mask128 = (u128)f.mask << f.shift;
        code = (code & ~mask128) | (((u128)v & f.mask) << f.shift);
    }
    std::string base_op = split(split(c.key, '_')[0], '.')[0];
    static const char* not_alu[] = {"LDG", "LDL", "LDS", "LDC", "LDCU", "STG", "STL", "STS", "ATOM", "RED", "BRA", "BSSY",
                                    "BSYNC", "EXIT", "RET", "BAR", "S2R", "S2UR", "LDSM", "LDGSTS", "QMMA"};
    bool is_alu = true;
    for (const char* n : not_alu) if (base_op == n) is_alu = false;
    if (is_alu) {
        const int bits[4] = {63, 62, 72, 73};
        for (int k = 0; k < 4; ++k) {
            if (!((synth >> k) & 1)) continue;
            bool covered = false;
            for (const Field& f : e.fields) covered |= (int)f.shift <= bits[k] && bits[k] < (int)(f.shift + f.bits);
            if (covered || ((e.and_base >> bits[k]) & 1)) continue;
            code |= (u128)1 << bits[k];
        }
    }
    bool full = false, lo3 = false, neg15 = false;
    for (const Field& f : e.fields) {
        if (f.shift <= 12 && f.shift + f.bits >= 16 && f.ext == X::Guard) full = true;
        if (f.shift <= 14 && f.shift + f.bits >= 15 && (f.ext == X::Guard || f.ext == X::GuardLo3)) lo3 = true;
        if (f.shift == 15 && f.bits == 1 && (f.ext == X::GuardNeg || f.ext == X::Inv || f.ext == X::Neg)) neg15 = true;
    }
    if (!(full || (lo3 && neg15))) code = (code & ~((u128)0xF << 12)) | ((u128)(guard & 0xF) << 12);
    {
        std::string mnemonic = split(c.key, '_')[0];
        for (const std::string& m : split(c.mod_group, ',')) mnemonic += "." + m;
        if (base_op == "QMMA" && contains(mnemonic, ".SP")) code &= ~((u128)1 << 80);
    }
    {
        const uint32_t slot_shift[3] = {24, 32, 64};
        std::vector<int> explicit_toks;
        for (const Field& f : e.fields) if (f.ext == X::Reuse) explicit_toks.push_back(f.token_idx);
        for (int i = 0; i < 3; ++i) {
            const Field* slot = nullptr;
            for (const Field& f : e.fields)
                if (f.shift == slot_shift[i] && f.bits == 8 && (f.ext == X::Reg || f.ext == X::UReg || f.ext == X::URegFf || f.ext == X::RegFf)) {
                    slot = &f;
                    break;
                }
            if (!slot) continue;
            if (std::find(explicit_toks.begin(), explicit_toks.end(), slot->token_idx) != explicit_toks.end()) continue;
            if ((reuse3 >> i) & 1) code |= (u128)1 << (122 + i);
            else code &= ~((u128)1 << (122 + i));
        }
    }
    const uint32_t epoch_static = ke.has_epoch ? ke.epoch : 0x000fc200u;
    const uint32_t epoch_default = 0x000fc200u, sched_field = 0x03FFFE00u;
    const uint32_t current_upper = (uint32_t)(code >> 96);
    const bool is_static = ke.has_class && (ke.ctrl_class == "exit_static" || ke.ctrl_class == "ctrl_flow" || ke.ctrl_class == "barrier");
    const bool is_nop = ke.has_class && ke.ctrl_class == "nop";
    const uint32_t reuse_bits = current_upper & 0x1C000000u;
    const uint32_t sched = (sched17 & 0x1FFFF) << 9;
    uint32_t upper;
    if (is_nop) upper = (epoch_static & ~sched_field) | reuse_bits | sched;
    else if (is_static) upper = epoch_static | reuse_bits;
    else upper = (epoch_default & ~sched_field) | reuse_bits | sched;
    return ((u128)upper << 96) | (code & (((u128)1 << 96) - 1));
}

u128 encode_from_record(const Oracle& o, uint16_t form, const uint32_t slots[8], uint32_t ctrl) {
    if (form >= o.by_variant.size()) return 0;
    const Candidate& c = *o.by_variant[form];
    const Entry& e = *o.table.get(c.key, c.mod_group);
    Layout L = slot_layout(e);
    std::vector<uint64_t> values;
    for (size_t i = 0; i < e.fields.size(); ++i)
        values.push_back(L.pos[i] == NOT_STORED ? 0 : get_bits(slots, L.pos[i], L.stored[i]));
    return orc_encode_record(o, form, values, (ctrl >> 24) & 0xF, (ctrl >> 20) & 0xF, (ctrl >> 17) & 7, ctrl & 0x1FFFF);
}

// Faithfulness check of reference src/main.rs:270, :578-581 at record level.
uint8_t roundtrip_status(const Oracle& o, u128 code) {
    uint16_t form; uint32_t slots[8], ctrl;
    decode_to_record(o, code, &form, slots, &ctrl);
    if ((ctrl >> 30) != 0) return 2;
    const u128 m = (u128)0x1FFFF << 105;
    return (encode_from_record(o, form, slots, ctrl) & ~m) == (code & ~m) ? 0 : 1;
}

// ---------------------------------------------------------------------------------------
// Synthetic stream (no counterpart in the reference; its corpus is private)
// ---------------------------------------------------------------------------------------

uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
uint64_t draw(uint64_t seed, uint64_t i, uint64_t j) {
    return splitmix64(seed * 0x9E3779B97F4A7C15ull + i * 0xD1342543DE82EF95ull + j);
}

struct Mix {
    std::vector<uint64_t> cdf;
    std::vector<std::string> key_at_rank;
};

Mix build_mix(const Oracle& o, uint32_t kind, uint64_t seed) {
    std::vector<std::string> keys;
    for (const auto& kv : o.table.entries)
        if (!kv.second.mod_groups.empty()) keys.push_back(kv.first);
    const size_t n = keys.size();
    Mix m;
    m.cdf.resize(n);
    const u128 total = (u128)1 << 64;
    if (kind == 0) {
        m.key_at_rank = keys;
        for (size_t r = 0; r < n; ++r) m.cdf[r] = (uint64_t)(total * (r + 1) / n - 1);
    } else if (kind == 1) {
        for (size_t i = n - 1; i > 0; --i) std::swap(keys[i], keys[(size_t)(draw(seed, ~0ull, i) % (i + 1))]);
        m.key_at_rank = keys;
        double sum = 0;
        std::vector<double> w(n);
        for (size_t r = 0; r < n; ++r) { w[r] = std::pow((double)(r + 1), -1.1); sum += w[r]; }
        double cum = 0;
        uint64_t prev = 0;
        for (size_t r = 0; r < n; ++r) {
            cum += w[r];
            double frac = cum / sum;
            uint64_t thr = frac >= 1.0 ? ~0ull : (uint64_t)std::ldexp(frac, 64);
            if (thr > 0) --thr;
            if (thr < prev) thr = prev;
            m.cdf[r] = prev = thr;
        }
    } else {
        std::vector<std::string> grp[3];
        for (const std::string& k : keys) {
            std::string b = split(split(k, '_')[0], '.')[0];
            if (b == "QMMA" || b == "HMMA" || b == "IMMA") grp[0].push_back(k);
            else if (b == "LDG" || b == "LDS" || b == "STG" || b == "LDGSTS") grp[1].push_back(k);
            else grp[2].push_back(k);
        }
        const u128 mass[3] = {total * 40 / 100, total * 25 / 100, total - total * 40 / 100 - total * 25 / 100};
        u128 base = 0;
        size_t r = 0;
        for (int g = 0; g < 3; ++g) {
            for (size_t i = 0; i < grp[g].size(); ++i, ++r) {
                m.key_at_rank.push_back(grp[g][i]);
                m.cdf[r] = (uint64_t)(base + mass[g] * (i + 1) / grp[g].size() - 1);
            }
            if (!grp[g].empty()) base += mass[g];
        }
    }
    m.cdf[n - 1] = ~0ull;
    return m;
}

// Word i of the stream and, unless it is raw noise, the generator's own record.
u128 synth_word(const Oracle& o, const Mix& mix, uint64_t seed, uint32_t noise_ppm, uint64_t i, uint16_t* form,
                uint32_t slots[8], uint32_t* ctrl) {
    for (int s = 0; s < 8; ++s) slots[s] = 0;
    if (noise_ppm && draw(seed, i, 0) % 1000000ull < noise_ppm) {
        u128 w = ((u128)draw(seed, i, 2) << 64) | draw(seed, i, 1);
        *form = 0xFFFF;
        *ctrl = pack_ctrl(w, 0, false, 0);
        return w;
    }
    const uint64_t u = draw(seed, i, 1);
    size_t rank = (size_t)(std::lower_bound(mix.cdf.begin(), mix.cdf.end(), u) - mix.cdf.begin());
    const std::string& key = mix.key_at_rank[rank];
    const KeyEntry& ke = o.table.entries.at(key);
    auto git = ke.mod_groups.begin();
    std::advance(git, (long)(draw(seed, i, 2) % ke.mod_groups.size()));
    const Entry& e = git->second;
    const uint32_t variant = o.variant_of.at({key, git->first});
    const uint64_t rg = draw(seed, i, 3);
    const unsigned guard = (rg & 1) ? 7u : (unsigned)((rg >> 1) & 15);
    const uint64_t rc = draw(seed, i, 4);
    static const unsigned bars[7] = {0, 1, 2, 3, 4, 5, 7};
    const unsigned stall = rc & 15, yld = (rc >> 4) & 1, rbar = bars[(rc >> 8) % 7], wbar = bars[(rc >> 16) % 7];
    const unsigned wait = (rc >> 24) & 63, reuse3 = (rc >> 32) & 7;
    const unsigned sched = (wait << 11) | (rbar << 8) | (wbar << 5) | (yld << 4) | stall;
    std::vector<uint64_t> values;
    Layout L = slot_layout(e);
    for (size_t f = 0; f < e.fields.size(); ++f) {
        const Field& fd = e.fields[f];
        const uint64_t r = draw(seed, i, 8 + f);
        uint64_t v;
        switch (fd.ext) {
            case X::UReg: case X::URegFf: case X::URegShr: case X::SubUR: case X::SubURShr: v = (r >> 60) == 0 ? 255 : r % 64; break;
            case X::Pred: case X::GuardLo3: case X::Barrier: v = r % 8; break;
            case X::Reg: case X::RegFf: case X::RegShr: case X::SubR: case X::SubRShr: v = r % 256; break;
            default: v = r; break;
        }
        v &= fd.mask;
        if (fd.shift >= 96) v = 0;
        else if (fd.shift + fd.bits > 96 && 96 - fd.shift < 64) v &= (1ull << (96 - fd.shift)) - 1;
        if (L.pos[f] != NOT_STORED) put_bits(slots, L.pos[f], L.stored[f], v);
        values.push_back(v);
    }
    *form = (uint16_t)variant;
    *ctrl = sched | (reuse3 << 17) | (guard << 20);
    return orc_encode_record(o, variant, values, 0, guard, reuse3, sched);
}

u128 load_word(const uint8_t* p) {
    uint64_t lo, hi;
    memcpy(&lo, p, 8); memcpy(&hi, p + 8, 8);
    return ((u128)hi << 64) | lo;
}
void store_word(uint8_t* p, u128 w) {
    uint64_t lo = (uint64_t)w, hi = (uint64_t)(w >> 64);
    memcpy(p, &lo, 8); memcpy(p + 8, &hi, 8);
}

template <typename Fn>
void parallel_for(uint64_t n, int threads, Fn fn) {
    if (threads <= 1 || n < 1024) { fn(0, n); return; }
    std::vector<std::thread> th;
    for (int k = 0; k < threads; ++k) {
        uint64_t b = n * (uint64_t)k / (uint64_t)threads, e = n * (uint64_t)(k + 1) / (uint64_t)threads;
        th.emplace_back([=] { fn(b, e); });
    }
    for (auto& t : th) t.join();
}

thread_local std::string g_error;

}  // namespace

// ---------------------------------------------------------------------------------------
// C interface for ctypes
// ---------------------------------------------------------------------------------------

extern "C" {

const char* orc_last_error() { return g_error.c_str(); }

void* orc_load_text(const char* json_text, uint64_t len) {
    try {
        Oracle* o = new Oracle;
        o->table = load_table(std::string(json_text, len));
        o->index.build(o->table);
        for (const auto& kv : o->table.entries)
            for (const auto& gv : kv.second.mod_groups) {
                o->variant_of[{kv.first, gv.first}] = (uint32_t)o->names.size();
                o->names.push_back({kv.first, gv.first});
            }
        o->by_variant.resize(o->names.size());
        for (const auto& b : o->index.opcode_map)
            for (const Candidate& c : b.second) o->by_variant[c.variant] = &c;
        return o;
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

void* orc_load(const char* path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) { g_error = std::string("failed to read ") + path; return nullptr; }
    std::stringstream ss;
    ss << in.rdbuf();
    std::string text = ss.str();
    return orc_load_text(text.data(), text.size());
}

void orc_free(void* h) { delete (Oracle*)h; }

void orc_table_info(void* h, uint32_t* keys, uint32_t* groups) {
    Oracle* o = (Oracle*)h;
    *keys = (uint32_t)o->table.entries.size();
    *groups = (uint32_t)o->names.size();
}

int orc_variant_name(void* h, uint32_t variant, const char** key, const char** mod_group) {
    Oracle* o = (Oracle*)h;
    if (variant >= o->names.size()) return -1;
    *key = o->names[variant].first.c_str();
    *mod_group = o->names[variant].second.c_str();
    return 0;
}

// Full decode of one word: the per-field values as the reference reports them.
// values/shifts/bits/tokens hold up to `cap` entries; returns the number of table fields,
// or -1 / -2 for the two rejection cases.
int orc_decode_full(void* h, uint64_t lo, uint64_t hi, uint32_t* variant, uint64_t* values, uint32_t* shifts,
                    uint32_t* bits, int32_t* tokens, uint32_t cap, uint32_t* synth, uint32_t* sched5, uint32_t* tie,
                    uint32_t* score) {
    Oracle* o = (Oracle*)h;
    Decoded d = o->decode(((u128)hi << 64) | lo);
    sched5[0] = d.stall; sched5[1] = d.yield; sched5[2] = d.wbar; sched5[3] = d.rbar; sched5[4] = d.wait;
    if (d.status) return -d.status;
    *variant = d.variant; *synth = d.synth; *tie = d.tie; *score = (uint32_t)d.cand->score;
    for (size_t i = 0; i < d.values.size() && i < cap; ++i) {
        values[i] = d.values[i]; shifts[i] = d.entry->fields[i].shift; bits[i] = d.entry->fields[i].bits;
        tokens[i] = d.entry->fields[i].token_idx;
    }
    return (int)d.values.size();
}

// Opcode text of a variant's key.
int orc_variant_opcode(void* h, uint32_t variant, char* out, uint32_t cap) {
    Oracle* o = (Oracle*)h;
    if (variant >= o->names.size()) return -1;
    snprintf(out, cap, "%s", opcode_of_key(o->names[variant].first).c_str());
    return 0;
}

// Kernel metadata of one code blob; returns the number of EXIT offsets (up to `cap` are written).
int orc_kernel_meta(void* h, const uint8_t* code, uint64_t nbytes, uint32_t* max_reg, uint32_t* barrier_mask,
                    uint32_t* exit_offsets, uint32_t cap) {
    KernelMetaResult r = infer_kernel_meta(*(const Oracle*)h, code, nbytes);
    *max_reg = r.max_reg; *barrier_mask = r.barrier_mask;
    for (size_t i = 0; i < r.exit_offsets.size() && i < cap; ++i) exit_offsets[i] = r.exit_offsets[i];
    return (int)r.exit_offsets.size();
}

// Extraction spelling of field `i` of a variant, as decode reports it.
int orc_field_extraction(void* h, uint32_t variant, uint32_t i, char* out, uint32_t cap) {
    Oracle* o = (Oracle*)h;
    if (variant >= o->names.size()) return -1;
    const Entry* e = o->table.get(o->names[variant].first, o->names[variant].second);
    if (i >= e->fields.size()) return -1;
    std::string s = extraction_name(e->fields[i]);
    snprintf(out, cap, "%s", s.c_str());
    return 0;
}

void orc_decode_batch(void* h, const uint8_t* words, uint64_t n, uint16_t* form, uint32_t* slots, uint32_t* ctrl, int threads) {
    const Oracle* o = (const Oracle*)h;
    parallel_for(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint32_t s[8];
            decode_to_record(*o, load_word(words + 16 * i), &form[i], s, &ctrl[i]);
            for (int k = 0; k < 8; ++k) slots[(uint64_t)k * n + i] = s[k];
        }
    });
}

void orc_encode_batch(void* h, const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl, uint64_t n, uint8_t* words, int threads) {
    const Oracle* o = (const Oracle*)h;
    parallel_for(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint32_t s[8];
            for (int k = 0; k < 8; ++k) s[k] = slots[(uint64_t)k * n + i];
            store_word(words + 16 * i, encode_from_record(*o, form[i], s, ctrl[i]));
        }
    });
}

void orc_roundtrip_batch(void* h, const uint8_t* words, uint64_t n, uint8_t* status, int threads) {
    const Oracle* o = (const Oracle*)h;
    parallel_for(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) status[i] = roundtrip_status(*o, load_word(words + 16 * i));
    });
}

// words/form/slots/ctrl may each be null.
void orc_synth_batch(void* h, uint32_t mix_kind, uint64_t seed, uint32_t noise_ppm, uint64_t first, uint64_t n, uint8_t* words,
                     uint16_t* form, uint32_t* slots, uint32_t* ctrl, int threads) {
    const Oracle* o = (const Oracle*)h;
    const Mix mix = build_mix(*o, mix_kind, seed);
    const Mix* mp = &mix;
    parallel_for(n, threads, [=](uint64_t b, uint64_t e) {
        for (uint64_t i = b; i < e; ++i) {
            uint16_t f; uint32_t s[8], c;
            u128 w = synth_word(*o, *mp, seed, noise_ppm, first + i, &f, s, &c);
            if (words) store_word(words + 16 * i, w);
            if (form) form[i] = f;
            if (ctrl) ctrl[i] = c;
            if (slots) for (int k = 0; k < 8; ++k) slots[(uint64_t)k * n + i] = s[k];
        }
    });
}

// Text sections of a little-endian ELF64 (reference src/elf.rs:29-58).  Writes up to `cap`
// (offset, size) pairs and NUL-separated names; returns the count or -1.
int orc_elf_text_sections(const uint8_t* b, uint64_t len, uint64_t* offsets, uint64_t* sizes, uint32_t cap, char* names, uint64_t names_cap) {
    auto r16 = [&](uint64_t o) { return (uint64_t)b[o] | ((uint64_t)b[o + 1] << 8); };
    auto r32 = [&](uint64_t o) { return r16(o) | (r16(o + 2) << 16); };
    auto r64 = [&](uint64_t o) { return r32(o) | (r32(o + 4) << 32); };
    if (len < 64 || memcmp(b, "\177ELF", 4) || b[4] != 2 || b[5] != 1) return -1;
    uint64_t shoff = r64(0x28), shnum = r16(0x3C), shstr = r16(0x3E);
    if (!shoff) return 0;
    if (r16(0x3A) != 64 || shoff + 64 > len) return -1;
    if (shnum == 0) shnum = r64(shoff + 0x20);
    if (shstr == 0xFFFF) shstr = r32(shoff + 0x28);
    if (shoff + shnum * 64 > len || shstr >= shnum) return -1;
    uint64_t so = r64(shoff + 64 * shstr + 0x18), ss = r64(shoff + 64 * shstr + 0x20);
    if (so + ss > len) return -1;
    uint32_t count = 0;
    uint64_t name_at = 0;
    for (uint64_t i = 0; i < shnum; ++i) {
        uint64_t sh = shoff + 64 * i, no = r32(sh);
        if (no >= ss) continue;
        std::string nm;
        uint64_t p = so + no;
        while (p < so + ss && b[p]) nm.push_back((char)b[p++]);
        if (p >= so + ss) continue;
        if (!(nm == ".text" || starts_with(nm, ".text."))) continue;
        if (r32(sh + 4) != 1 || r64(sh + 0x20) == 0) continue;
        if (count < cap && name_at + nm.size() + 1 <= names_cap) {
            offsets[count] = r64(sh + 0x18); sizes[count] = r64(sh + 0x20);
            memcpy(names + name_at, nm.c_str(), nm.size() + 1);
            name_at += nm.size() + 1;
        }
        ++count;
    }
    return (int)count;
}

}  // extern "C"
