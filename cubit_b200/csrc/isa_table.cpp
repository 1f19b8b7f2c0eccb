#include "isa_table.hpp"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>

#include "json.hpp"

namespace cubit {

using cubit_json::Value;

static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) ++a;
    while (b > a && isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}

u128 parse_hex_u128(const std::string& raw) {
    std::string s = trim(raw);
    if (s.size() >= 2 && s[0] == '0' && (s[1] == 'x' || s[1] == 'X')) s = s.substr(2);
    if (s.empty()) throw std::runtime_error("invalid hex: " + raw);
    u128 v = 0;
    for (char c : s) {
        unsigned d;
        if (c >= '0' && c <= '9') d = unsigned(c - '0');
        else if (c >= 'a' && c <= 'f') d = unsigned(c - 'a' + 10);
        else if (c >= 'A' && c <= 'F') d = unsigned(c - 'A' + 10);
        else throw std::runtime_error("invalid hex: " + raw);
        if (v >> 124) throw std::runtime_error("invalid hex (wider than 128 bits): " + raw);
        v = (v << 4) | d;
    }
    return v;
}

std::string hex_u128(u128 v) {
    char buf[40];
    snprintf(buf, sizeof buf, "0x%016llx%016llx", (unsigned long long)(uint64_t)(v >> 64),
             (unsigned long long)(uint64_t)v);
    return buf;
}

static bool starts_with(const std::string& s, const char* p) { return s.compare(0, strlen(p), p) == 0; }

// Parses the decimal tail of "reg_shr3"-style spellings as a u8.
static uint8_t parse_u8_tail(const std::string& s, size_t from, const std::string& whole) {
    if (from >= s.size()) throw std::runtime_error("invalid extraction '" + whole + "'");
    unsigned v = 0;
    size_t i = from;
    if (s[i] == '+') ++i;
    if (i >= s.size()) throw std::runtime_error("invalid extraction '" + whole + "'");
    for (; i < s.size(); ++i) {
        if (s[i] < '0' || s[i] > '9') throw std::runtime_error("invalid extraction '" + whole + "'");
        v = v * 10 + unsigned(s[i] - '0');
        if (v > 255) throw std::runtime_error("invalid extraction '" + whole + "'");
    }
    return uint8_t(v);
}

// "sub_<tag><idx>_shr<s>" with tag in {r, ur, imm}.
static void parse_sub_shr(const std::string& s, const char* tag, uint8_t* idx, uint8_t* shr) {
    std::vector<std::string> parts;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, '_')) parts.push_back(item);
    if (!s.empty() && s.back() == '_') parts.push_back("");
    if (parts.size() < 3 || !starts_with(parts[1], tag) || !starts_with(parts[2], "shr"))
        throw std::runtime_error("invalid extraction '" + s + "'");
    *idx = parse_u8_tail(parts[1], strlen(tag), s);
    *shr = parse_u8_tail(parts[2], 3, s);
}

// Table spelling -> kind, numeric parameters and the spelling reported by decode.
static void parse_extraction(const std::string& s, IsaField* f) {
    struct Fixed { const char* in; Ext e; uint8_t p, p2; const char* out; };
    static const Fixed fixed[] = {
        {"guard", Ext::Guard, 0, 0, "guard"}, {"guard_lo3", Ext::GuardLo3, 0, 0, "guardlo3"},
        {"guard_neg", Ext::GuardNeg, 0, 0, "guardneg"}, {"reg", Ext::Reg, 0, 0, "reg"},
        {"ureg", Ext::UReg, 0, 0, "ureg"}, {"ureg_ff", Ext::URegFf, 0, 0, "ureg_ff"},
        {"reg_ff", Ext::RegFf, 0, 0, "reg_ff"}, {"pred", Ext::Pred, 0, 0, "pred"},
        {"upred", Ext::Pred, 0, 0, "pred"}, {"barrier", Ext::Barrier, 0, 0, "barrier"},
        {"imm", Ext::Imm, 0, 0, "imm"}, {"imm_dec", Ext::ImmDec, 0, 0, "immdec"},
        {"imm_dec_u32", Ext::ImmDecU32, 0, 0, "immdecu32"}, {"f32", Ext::F32, 0, 0, "f32"},
        {"f16", Ext::F16, 0, 0, "f16"}, {"f16_d", Ext::F16d, 0, 0, "f16_d"},
        {"f64hi", Ext::F64hi, 0, 0, "f64hi"}, {"neg", Ext::Neg, 0, 0, "neg"},
        {"neg_shl1", Ext::NegShl1, 0, 0, "negshl1"}, {"reuse", Ext::Reuse, 0, 0, "reuse"},
        {"inv", Ext::Inv, 0, 0, "inv"}, {"abs", Ext::Abs, 0, 0, "abs"},
        {"neg_abs", Ext::NegAbs, 0, 0, "negabs"}, {"byte_sel", Ext::ByteSel, 0, 0, "bytesel"},
        {"sysreg", Ext::SysReg, 0, 0, "sysreg"}, {"sysreg_lo7", Ext::SysRegLo7, 0, 0, "sysreglo7"},
        {"sysreg_lo4", Ext::SysRegLo4, 0, 0, "sysreglo4"}, {"sysreg_hi4", Ext::SysRegHi4, 0, 0, "sysreghi4"},
        {"sysreg_hi1", Ext::SysRegHi1, 0, 0, "sysreghi1"},
        {"sub_r0", Ext::SubR, 0, 0, "sub_r0"}, {"sub_r1", Ext::SubR, 1, 0, "sub_r1"},
        {"sub_r2", Ext::SubR, 2, 0, "sub_r2"}, {"sub_ur0", Ext::SubUR, 0, 0, "sub_ur0"},
        {"sub_ur1", Ext::SubUR, 1, 0, "sub_ur1"}, {"sub_imm0", Ext::SubImm, 0, 0, "sub_imm0"},
        {"sub_imm1", Ext::SubImm, 1, 0, "sub_imm1"}, {"sub_imm2", Ext::SubImm, 2, 0, "sub_imm2"},
        {"sub_imm0_s24", Ext::SubImmS24, 0, 0, "sub_imm0_s24"},
        {"sub_imm1_s24", Ext::SubImmS24, 1, 0, "sub_imm1_s24"},
        {"sub_imm2_s24", Ext::SubImmS24, 2, 0, "sub_imm2_s24"},
        {"cm16_off", Ext::Cm16Off, 0, 0, "cm16off"}, {"cm17_off", Ext::Cm17Off, 0, 0, "cm17off"},
        {"opaque_mod", Ext::OpaqueModifier, 0, 0, "opaque_mod"}, {"", Ext::None, 0, 0, "none"},
    };
    for (const Fixed& fx : fixed) {
        if (s == fx.in) {
            f->ext = fx.e; f->param = fx.p; f->param2 = fx.p2; f->ext_name = fx.out;
            return;
        }
    }
    // Parameterised spellings, tried in the reference's order (src/table.rs:135-180).
    if (starts_with(s, "reg_shr")) {
        f->ext = Ext::RegShr; f->param = parse_u8_tail(s, 7, s);
        f->ext_name = "reg_shr" + std::to_string(f->param);
        return;
    }
    if (starts_with(s, "ureg_shr")) {
        f->ext = Ext::URegShr; f->param = parse_u8_tail(s, 8, s);
        f->ext_name = "ureg_shr" + std::to_string(f->param);
        return;
    }
    if (starts_with(s, "imm_shr")) {
        f->ext = Ext::ImmShr; f->param = parse_u8_tail(s, 7, s);
        f->ext_name = "imm_shr" + std::to_string(f->param);
        return;
    }
    const bool has_shr = s.find("_shr") != std::string::npos;
    if (starts_with(s, "sub_r") && has_shr) {
        f->ext = Ext::SubRShr; parse_sub_shr(s, "r", &f->param, &f->param2);
        f->ext_name = "sub_r" + std::to_string(f->param) + "_shr" + std::to_string(f->param2);
        return;
    }
    if (starts_with(s, "sub_ur") && has_shr) {
        f->ext = Ext::SubURShr; parse_sub_shr(s, "ur", &f->param, &f->param2);
        f->ext_name = "sub_ur" + std::to_string(f->param) + "_shr" + std::to_string(f->param2);
        return;
    }
    if (starts_with(s, "sub_imm") && has_shr) {
        f->ext = Ext::SubImmShr; parse_sub_shr(s, "imm", &f->param, &f->param2);
        f->ext_name = "sub_imm" + std::to_string(f->param) + "_shr" + std::to_string(f->param2);
        return;
    }
    throw std::runtime_error("unknown extraction '" + s + "'");
}

static uint32_t json_u32(const Value* v, const char* what, const std::string& where) {
    if (!v || v->kind != Value::Number || !v->is_integer || v->is_negative || v->mag > 0xFFFFFFFFull)
        throw std::runtime_error(std::string("failed to parse table JSON: ") + what + " of " + where +
                                 " is not a u32");
    return uint32_t(v->mag);
}
static int32_t json_i32(const Value* v, const char* what, const std::string& where) {
    if (!v || v->kind != Value::Number || !v->is_integer ||
        (!v->is_negative && v->mag > 0x7FFFFFFFull) || (v->is_negative && v->mag > 0x80000000ull))
        throw std::runtime_error(std::string("failed to parse table JSON: ") + what + " of " + where +
                                 " is not an i32");
    return v->is_negative ? int32_t(-(int64_t)v->mag) : int32_t(v->mag);
}

// One "mod_groups" member -> variant (reference src/table.rs:353-396).
static IsaVariant parse_mod_group(const std::string& key, const std::string& mods, const Value& g) {
    const std::string where = key + "::" + mods;
    if (!g.is_object()) throw std::runtime_error("failed to parse table JSON: " + where + " is not an object");
    const Value* ab = g.get("and_base");
    if (!ab || !ab->is_string())
        throw std::runtime_error("failed to parse table JSON: missing and_base for " + where);
    const Value* fl = g.get("fields");
    if (!fl || !fl->is_array())
        throw std::runtime_error("failed to parse table JSON: missing fields for " + where);
    IsaVariant v;
    v.mod_group = mods;
    try {
        v.and_base = parse_hex_u128(ab->str);
    } catch (const std::exception& e) {
        throw std::runtime_error("bad and_base for " + where + ": " + e.what());
    }
    for (const Value& jf : fl->arr) {
        if (!jf.is_object()) throw std::runtime_error("failed to parse table JSON: field of " + where);
        IsaField f;
        f.shift = json_u32(jf.get("shift"), "shift", where);
        f.bits = json_u32(jf.get("bits"), "bits", where);
        f.token_idx = json_i32(jf.get("token_idx"), "token_idx", where);
        const Value* ex = jf.get("extraction");
        if (!ex || !ex->is_string())
            throw std::runtime_error("failed to parse table JSON: extraction of " + where);
        uint64_t end = uint64_t(f.shift) + uint64_t(f.bits);
        if (end > 0xFFFFFFFFull)
            throw std::runtime_error("field range overflow for " + where + ": shift=" +
                                     std::to_string(f.shift) + ", bits=" + std::to_string(f.bits));
        if (f.bits == 0 || end > 128)
            throw std::runtime_error("field outside 128-bit instruction for " + where + ": shift=" +
                                     std::to_string(f.shift) + ", bits=" + std::to_string(f.bits));
        f.mask = f.bits >= 64 ? ~0ull : ((1ull << f.bits) - 1);
        try {
            parse_extraction(ex->str, &f);
        } catch (const std::exception& e) {
            throw std::runtime_error("bad extraction for " + where + " at shift " +
                                     std::to_string(f.shift) + ": " + e.what());
        }
        v.fields.push_back(std::move(f));
    }
    const Value* vm = g.get("variable_mask");
    if (vm && vm->kind != Value::Null) {
        if (!vm->is_string())
            throw std::runtime_error("failed to parse table JSON: variable_mask of " + where);
        try {
            v.variable_mask = parse_hex_u128(vm->str);
        } catch (const std::exception& e) {
            throw std::runtime_error("bad variable_mask for " + where + ": " + e.what());
        }
    } else {
        u128 m = 0;
        for (const IsaField& f : v.fields) m |= f.range();
        v.variable_mask = m;
    }
    return v;
}

// Last occurrence wins for repeated member names; iteration is bytewise sorted.
static std::map<std::string, const Value*> sorted_members(const Value& obj) {
    std::map<std::string, const Value*> out;
    for (const auto& m : obj.obj) out[m.first] = &m.second;
    return out;
}

static CtrlKind ctrl_kind_of(const std::string& cc) {
    if (cc == "nop") return CTRL_NOP;
    if (cc == "exit_static" || cc == "ctrl_flow" || cc == "barrier") return CTRL_STATIC;
    return CTRL_NORMAL;
}

IsaTable IsaTable::from_json_text(const std::string& text) {
    Value root;
    try {
        root = cubit_json::parse(text);
    } catch (const std::exception& e) {
        throw std::runtime_error(std::string("invalid JSON: ") + e.what());
    }
    const bool unified = text.find("\"_meta\"") != std::string::npos &&
                         text.find("\"instructions\"") != std::string::npos;
    if (!root.is_object()) throw std::runtime_error("failed to parse table JSON: top level is not an object");

    // ctrl_class name -> epoch upper32 (reference src/table.rs:312-343).
    std::map<std::string, uint32_t> epoch_of_class;
    const Value* instructions = &root;
    if (unified) {
        instructions = root.get("instructions");
        if (!instructions || !instructions->is_object()) throw std::runtime_error("missing 'instructions' key");
        if (const Value* meta = root.get("_meta")) {
            std::map<std::string, uint32_t> epochs;
            const Value* ce = meta->get("ctrl_epochs");
            if (ce && ce->is_object())
                for (const auto& kv : sorted_members(*ce)) {
                    const Value* up = kv.second->get("upper32");
                    if (up && up->is_string()) {
                        try { epochs[kv.first] = uint32_t(parse_hex_u128(up->str)); } catch (...) {}
                    }
                }
            const Value* cc = meta->get("ctrl_classes");
            if (cc && cc->is_object())
                for (const auto& kv : sorted_members(*cc)) {
                    const Value* en = kv.second->get("hi_upper32");
                    if (en && en->is_string()) {
                        auto it = epochs.find(en->str);
                        if (it != epochs.end()) epoch_of_class[kv.first] = it->second;
                    }
                }
        }
    }

    IsaTable t;
    for (const auto& kv : sorted_members(*instructions)) {
        const std::string& key = kv.first;
        const Value& entry = *kv.second;
        const Value* groups = entry.get("mod_groups");
        if (!groups) {
            if (unified) continue;   // unified entries without encodings are skipped
            throw std::runtime_error("failed to parse table JSON: missing mod_groups for " + key);
        }
        if (!groups->is_object())
            throw std::runtime_error("failed to parse table JSON: mod_groups of " + key + " is not an object");
        IsaKey k;
        k.name = key;
        if (unified) {
            const Value* cc = entry.get("ctrl_class");
            if (cc && cc->is_string()) {
                k.has_ctrl_class = true;
                k.ctrl_class = cc->str;
                k.ctrl_kind = ctrl_kind_of(cc->str);
                auto it = epoch_of_class.find(cc->str);
                if (it != epoch_of_class.end()) { k.has_epoch = true; k.epoch_upper32 = it->second; }
            }
        }
        k.first_variant = uint32_t(t.variants.size());
        const uint32_t key_id = uint32_t(t.keys.size());
        for (const auto& g : sorted_members(*groups)) {
            IsaVariant v = parse_mod_group(key, g.first, *g.second);
            v.key_id = key_id;
            t.variants.push_back(std::move(v));
        }
        k.n_variants = uint32_t(t.variants.size()) - k.first_variant;
        t.keys.push_back(std::move(k));
    }
    return t;
}

IsaTable IsaTable::from_file(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("failed to read " + path);
    std::stringstream ss;
    ss << in.rdbuf();
    return from_json_text(ss.str());
}

}  // namespace cubit
