#include "flat_table.hpp"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <tuple>

#include "codec_core.cuh"

namespace cubit {

// ---- string helpers over instruction keys -----------------------------------------------

static std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    size_t a = 0;
    for (;;) {
        size_t b = s.find(sep, a);
        if (b == std::string::npos) { out.push_back(s.substr(a)); return out; }
        out.push_back(s.substr(a, b - a));
        a = b + 1;
    }
}
static bool starts_with(const std::string& s, const char* p) { return s.compare(0, strlen(p), p) == 0; }
static bool ends_with(const std::string& s, const char* p) {
    size_t n = strlen(p);
    return s.size() >= n && s.compare(s.size() - n, n, p) == 0;
}
static bool contains(const std::string& s, const char* p) { return s.find(p) != std::string::npos; }
static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) ++a;
    while (b > a && isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}

// Operand-type tokens that can follow the opcode in a key (reference src/decoder.rs:602-607).
static bool is_op_type(const std::string& p) {
    static const char* kTypes[] = {"ARURR", "ARURI", "ARUR", "AURI", "AURR", "AUR", "cAI", "dARI", "ARI", "UP", "UR",
                                   "SR",    "FI",    "II",   "IM",   "LO",   "R",   "P",   "L",    "B",   "?"};
    for (const char* t : kTypes)
        if (p == t) return true;
    return false;
}
static std::vector<std::string> operand_types(const std::string& key) {
    std::vector<std::string> out;
    bool in_ops = false;
    for (const std::string& part : split(key, '_')) {
        if (!in_ops && is_op_type(part)) in_ops = true;
        if (in_ops) out.push_back(part);
    }
    return out;
}
static bool is_pred_type(const std::string& t) { return t == "P" || t == "UP"; }
static std::string base_op_of(const std::string& key) {
    std::string first = split(key, '_')[0];
    return split(first, '.')[0];
}

// How well the field token assignments agree with the operand types named by the key
// (reference src/decoder.rs:623-666).  The loader folds "upred" into Pred, so the
// reference's upred arms can never fire and are absent here.
static int consistency_score(const std::string& key, const IsaVariant& v) {
    const std::vector<std::string> types = operand_types(key);
    int score = 0;
    for (const IsaField& f : v.fields) {
        if (f.token_idx <= 0) continue;
        const size_t idx = size_t(f.token_idx - 1);
        const std::string t = idx < types.size() ? types[idx] : std::string();
        const std::string& e = f.ext_name;
        const bool is_pred = e == "pred" || e == "guard";
        const bool is_reg = e == "reg" || e == "ureg" || e == "ureg_ff" || e == "reg_ff" || e == "reg_shr1" ||
                            e == "reg_shr2" || e == "reg_shr3";
        const bool is_imm = starts_with(e, "imm") || e == "f32" || e == "f16" || e == "f16_d" || e == "f64hi";
        const bool is_barrier = e == "barrier";
        const bool want_pred = t == "P", want_upred = t == "UP", want_reg = t == "R" || t == "UR";
        const bool want_imm = t == "II" || t == "IM" || t == "LO" || t == "FI", want_barrier = t == "B";
        if (want_pred && is_pred) score += 2;
        else if (want_barrier && is_barrier) score += 4;
        else if (want_upred && is_pred) score -= 2;
        else if ((want_reg && is_reg) || (want_imm && is_imm)) score += 2;
        else if ((want_pred && is_reg) || (want_reg && is_pred)) score -= 5;
        else if (want_reg && is_imm) score -= 4;
        else if (want_imm && is_reg) score -= 2;
        else if (want_barrier && is_pred) score -= 5;
        if ((t == "dARI" || t == "ARURI") && starts_with(e, "sub_ur")) score += 3;
    }
    return score;
}

static bool names_mode_in_opcode(const std::string& key, const char* mode) {
    std::vector<std::string> dotted = split(split(key, '_')[0], '.');
    for (size_t i = 1; i < dotted.size(); ++i)
        if (dotted[i] == mode) return true;
    return false;
}
static bool names_mode_in_group(const std::string& mods, const char* mode) {
    for (const std::string& m : split(mods, ','))
        if (trim(m) == mode) return true;
    return false;
}

static std::string field_display_name(const IsaField& f) {
    if (f.bits == 8 && f.shift == 16) return "Rd";
    if (f.bits == 8 && f.shift == 24) return "Ra";
    if (f.bits == 8 && f.shift == 32) return "Rb";
    if (f.bits == 8 && f.shift == 64) return "Rc";
    if (f.bits == 4 && f.shift == 12) return "guard";
    return "[" + std::to_string(f.shift + f.bits - 1) + ":" + std::to_string(f.shift) + "]";
}

// Opcode = key segments before the first operand type; "B" right after a ...PACK segment
// is a lane suffix and stays in the opcode (reference src/decoder.rs:357-371).
static std::string opcode_of(const std::string& key) {
    std::vector<std::string> parts = split(key, '_'), op;
    for (const std::string& p : parts) {
        if (is_op_type(p)) {
            const bool pack_b = p == "B" && !op.empty() && ends_with(op.back(), "PACK");
            if (!pack_b) break;
        }
        op.push_back(p);
    }
    if (op.empty()) return parts[0];
    std::string out = op[0];
    for (size_t i = 1; i < op.size(); ++i) out += "_" + op[i];
    return out;
}

static uint32_t limb(u128 v, int k) { return uint32_t(v >> (32 * k)); }
static int popcount128(u128 v) { return __builtin_popcountll(uint64_t(v)) + __builtin_popcountll(uint64_t(v >> 64)); }

static uint32_t gen_class(const IsaField& f) {
    switch (f.ext) {
        case Ext::UReg: case Ext::URegFf: case Ext::URegShr: case Ext::SubUR: case Ext::SubURShr: return GC_UREG;
        case Ext::Pred: case Ext::GuardLo3: case Ext::Barrier: return GC_MOD8;
        case Ext::Reg: case Ext::RegFf: case Ext::RegShr: case Ext::SubR: case Ext::SubRShr: return GC_REG;
        default: return GC_UNIFORM;
    }
}

namespace {

struct Static {
    u128 smask = 0, sbase = 0, bmask = 0, bbase = 0, base96 = 0;
    bool s_ok = false, b_ok = false;
    int score = 0;
    std::tuple<int, int, int, int, int> mid;   // opaque, plain-address, undiscovered, length, -score
    std::tuple<int, int> lo;                   // -popcount(match), -len(mod_group)
    uint32_t flags = 0;
    u128 weakest() const { return b_ok ? bmask : smask; }
    bool matchable() const { return s_ok || b_ok; }
};

struct TreeBuilder {
    const std::vector<Static>& st;
    const std::vector<uint32_t>& ext_of;   // variant -> extraction record index
    FlatTable& ft;
    uint32_t max_depth = 0;
    size_t class_budget = 0;   // bit-node splits stop once this many class records exist
    std::map<std::pair<u128, u128>, uint32_t> broad_index;   // identical broad records are stored once

    // A class: variants with identical masks, constant bits and and_base.
    typedef std::tuple<bool, u128, u128, bool, u128, u128, u128> ClassKey;
    ClassKey class_key(uint32_t v) const {
        const Static& s = st[v];
        return ClassKey(s.s_ok, s.s_ok ? s.smask : 0, s.s_ok ? s.sbase : 0, s.b_ok, s.b_ok ? s.bmask : 0,
                        s.b_ok ? s.bbase : 0, s.base96);
    }
    size_t class_count(const std::vector<uint32_t>& vs) const {
        std::map<ClassKey, int> seen;
        for (uint32_t v : vs) seen[class_key(v)] = 1;
        return seen.size();
    }

    uint32_t make_leaf(const std::vector<uint32_t>& vs) {
        // Rank keys are dense inside the leaf: only its candidates are ever compared.
        std::map<std::tuple<int, int, int, int, int>, uint32_t> mid_rank;
        std::map<std::tuple<int, int>, uint32_t> lo_rank;
        for (uint32_t v : vs) { mid_rank[st[v].mid] = 0; lo_rank[st[v].lo] = 0; }
        uint32_t r = 0;
        for (auto& kv : mid_rank) kv.second = r++;
        r = 0;
        for (auto& kv : lo_rank) kv.second = r++;
        if (mid_rank.size() > 128 || lo_rank.size() > 128 || vs.size() > 256)
            throw std::runtime_error("a leaf of the match tree has too many candidates for 32-bit rank keys");
        std::map<uint32_t, uint32_t> key_of;   // variant -> static key; vs is in canonical order
        for (size_t i = 0; i < vs.size(); ++i) {
            const Static& s = st[vs[i]];
            key_of[vs[i]] = (uint32_t(s.score < 0 ? 1 : 0) << 31) | (mid_rank[s.mid] << 22) | (lo_rank[s.lo] << 8) | uint32_t(i);
        }

        // Choice flags that no rule can ask for inside this leaf are dropped from its records, so that they
        // do not show up as "carried by some candidate but not by the top one" and send the kernel into
        // the rule choice for nothing: the LEA flags without a LEA form among the candidates, the _UP flag
        // without a uniform LOP3 form, the branch-mode flags without a BRA form, and "no middle predicate"
        // when every candidate has it (the rule asks for it only when the top candidate lacks it).
        uint32_t strip = 0;
        {
            bool lea = false, ulop3 = false, bra = false, all_no_mid = true;
            for (uint32_t v : vs) {
                const uint32_t f = st[v].flags;
                lea |= (f & FL1_IS_LEA) != 0; ulop3 |= (f & FL1_IS_ULOP3) != 0; bra |= (f & FL_IS_BRA) != 0;
                all_no_mid &= (f & FL_NO_MID_P) != 0;
            }
            if (!lea) strip |= FL_LEA_A1 | FL_LEA_A2;
            if (!ulop3) strip |= FL_ENDS_UP;
            if (!bra) strip |= FL_EXP_U | FL_EXP_DIV | FL_EXP_CONV | FL_GRP_U | FL_GRP_DIV | FL_GRP_CONV | FL_BRA_NOMODE;
            if (all_no_mid) strip |= FL_NO_MID_P;
            // Word bits that every candidate of the leaf demands with the same value hold for every word that
            // matches any of them; a rule whose condition they contradict never fires here.
            u128 fixed = 0, value = 0;
            bool seen = false;
            for (uint32_t v : vs) {
                const Static& c = st[v];
                if (!c.matchable()) continue;
                const u128 m = c.weakest(), b = c.b_ok ? c.bbase : c.sbase;
                if (!seen) { fixed = m; value = b; seen = true; }
                else fixed &= m & ~(value ^ b);
            }
            auto one = [&](int bit) { return ((fixed >> bit) & 1) && ((value >> bit) & 1); };
            auto zero = [&](int bit) { return ((fixed >> bit) & 1) && !((value >> bit) & 1); };
            if (one(87) && one(88) && one(89)) strip |= FL_HAS_TP | FL_LEA_A1 | FL_LEA_A2;   // never a real trailing predicate
            if (one(81) && one(82) && one(83)) strip |= FL_HAS_OUTPRED_F | FL_LEA_A1;        // the output slot always reads PT
            if (zero(81) || zero(82) || zero(83)) strip |= FL_NO_MID_P | FL_LEA_A2;          // ... never reads PT
            for (int bit = 64; bit < 72; ++bit)
                if (zero(bit)) strip |= FL_SHL_OK;                                           // Rc is never RZ
            bool r2_possible = false;
            for (uint32_t v : vs) {
                const uint32_t f = st[v].flags;
                if (!(f & FL1_HAS_R2)) continue;
                const int lo = 80 + int((f >> FL1_R2_SHIFT_POS) & 7u), n = 1 + int((f >> FL1_R2_BITS_POS) & 15u);
                bool can = true;
                for (int bit = lo; bit < lo + n; ++bit) can &= !zero(bit);
                r2_possible |= can;
            }
            if (!r2_possible) strip |= FL_NO_OUTPRED;                                        // no output-predicate field can read all ones
            if (one(32) || one(33)) strip |= FL_BRA_NOMODE;                                  // the branch mode is never 0
            if (zero(32) && zero(33)) strip |= FL_EXP_U | FL_EXP_DIV | FL_EXP_CONV | FL_GRP_U | FL_GRP_DIV | FL_GRP_CONV;
            if (zero(32) || one(33)) strip |= FL_EXP_U | FL_GRP_U;                           // mode 1 is .U, 2 .DIV, 3 .CONV
            if (one(32) || zero(33)) strip |= FL_EXP_DIV | FL_GRP_DIV;
            if (zero(32) || zero(33)) strip |= FL_EXP_CONV | FL_GRP_CONV;
        }
        auto flags_of = [&](uint32_t v) { return st[v].flags & ~strip; };
        std::map<ClassKey, std::vector<uint32_t>> groups;
        std::vector<ClassKey> order;   // classes in order of their first (canonical) member
        for (uint32_t v : vs) {
            ClassKey k = class_key(v);
            if (!groups.count(k)) order.push_back(k);
            groups[k].push_back(v);
        }
        const uint32_t first_class = uint32_t(ft.classes.size() / CR_WORDS);
        if (order.size() > 255 || first_class + order.size() >= (1u << 20)) throw std::runtime_error("leaf too large");
        // Members in rank order inside a class; classes in rank order of their best member.
        for (auto& kv : groups)
            std::sort(kv.second.begin(), kv.second.end(), [&](uint32_t a, uint32_t b) { return key_of[a] < key_of[b]; });
        // Static rank order of classes.  Two strictly matching classes compare by
        // (score sign, middle rank, popcount(and_base & word), low rank, canonical position).  The
        // popcount splits into a constant part under the strict mask and a word-dependent part
        // over and_base bits outside it (mostly baked guard bits); classes with the *same* outside
        // bits get the same word-dependent part, so their order is static.
        auto sort_key = [&](const ClassKey& c) {
            const uint32_t v = groups[c][0], k = key_of[v];
            const Static& b = st[v];
            const int pst = b.s_ok ? popcount128(b.base96 & b.smask) : 0;
            return std::make_tuple(k >> 22, -pst, k & 0x7FFFu);
        };
        std::sort(order.begin(), order.end(), [&](const ClassKey& a, const ClassKey& b) { return sort_key(a) < sort_key(b); });
        // CR_GROUP: classes whose order against this one is NOT settled by position — same
        // (score sign, middle rank) and either different outside bits (word-dependent) or an
        // identical static tuple (a tie the ranking loop has to report).
        auto outside = [&](const ClassKey& c) { const Static& b = st[groups[c][0]]; return b.s_ok ? (b.base96 & ~b.smask) : ~(u128)0; };
        // Two classes whose strict masks demand different values of some bit never match the same word strictly.
        auto can_both_match = [&](const ClassKey& a, const ClassKey& b) {
            const Static& x = st[groups[a][0]];
            const Static& y = st[groups[b][0]];
            return !x.s_ok || !y.s_ok || ((x.sbase ^ y.sbase) & x.smask & y.smask) == 0;
        };
        auto unsettled = [&](const ClassKey& a, const ClassKey& b) {
            const auto ka = sort_key(a), kb = sort_key(b);
            if (std::get<0>(ka) != std::get<0>(kb)) return false;
            if (!st[groups[a][0]].s_ok || !st[groups[b][0]].s_ok) return true;
            if (!can_both_match(a, b)) return false;   // never strict matches of the same word
            // x beats y on every word when the constant part of its popcount leads by more than y's and_base
            // bits outside the masks can make up for, or leads by exactly that much and its low rank is better
            // (an equal low rank is a tie the ranking loop has to report).
            auto always_beats = [&](const ClassKey& x, const ClassKey& y, const std::tuple<uint32_t, int, uint32_t>& kx,
                                    const std::tuple<uint32_t, int, uint32_t>& ky) {
                const int lead = -std::get<1>(kx) + std::get<1>(ky) - popcount128(outside(y) & ~outside(x));
                return lead > 0 || (lead == 0 && (std::get<2>(kx) >> 8) < (std::get<2>(ky) >> 8));
            };
            return !always_beats(a, b, ka, kb) && !always_beats(b, a, kb, ka);
        };
        std::vector<uint32_t> leaf_group(order.size()), leaf_key(order.size()), leaf_within(order.size());
        uint32_t leaf_broad16 = 0;   // which of the first 16 classes have a broad record
        bool leaf_has_broad = false;
        for (size_t ci = 0; ci < order.size(); ++ci) {
            const ClassKey& ck = order[ci];
            std::vector<uint32_t>& mem = groups[ck];
            if (mem.size() > 255) throw std::runtime_error("class too large");
            uint32_t group_mask = 0;
            for (size_t cj = 0; cj < order.size() && cj < 32; ++cj)
                if (cj == ci || unsettled(order[cj], ck)) group_mask |= 1u << cj;
            const Static& best = st[mem[0]];
            uint32_t rec[CR_WORDS] = {0};
            for (int k = 0; k < 3; ++k) {
                // A side that can never match gets mask 0 / base bit 16: (cc & 0) ^ base is never 0.  Bits 15:0
                // of limb 0 are not part of the test (the word's are cleared first): bits 11:0 chose the directory
                // entry, bits 15:12 are the guard, which no mask holds.
                rec[CR_SMASK + k] = best.s_ok ? uint32_t(best.smask >> (32 * k)) : 0;
                rec[CR_SBASE + k] = best.s_ok ? uint32_t(best.sbase >> (32 * k)) : (k == 0 ? 0x10000u : 0u);
                rec[CR_BASE + k] = uint32_t(best.base96 >> (32 * k));
            }
            if (rec[CR_SMASK] & 0xF000u) throw std::runtime_error("internal: a strict mask holds guard bits");
            rec[CR_SMASK] &= 0xFFFF0000u;
            rec[CR_SBASE] &= 0xFFFF0000u;
            uint32_t info = mem.size() > 1 ? uint32_t(CI_SEVERAL) : 0u;
            // The broad test only adds something when it can succeed where the strict one fails.
            if (best.b_ok && !(best.s_ok && best.bmask == best.smask)) {
                auto found = broad_index.find({best.bmask, best.bbase});
                if (found == broad_index.end()) {
                    const uint32_t bi = uint32_t(ft.broad.size() / BR_WORDS);
                    if (bi > CI_BROAD_MASK) throw std::runtime_error("too many broad records");
                    uint32_t br[BR_WORDS] = {0};
                    for (int k = 0; k < 3; ++k) { br[k] = uint32_t(best.bmask >> (32 * k)); br[3 + k] = uint32_t(best.bbase >> (32 * k)); }
                    ft.broad.insert(ft.broad.end(), br, br + BR_WORDS);
                    found = broad_index.emplace(std::make_pair(best.bmask, best.bbase), bi).first;
                }
                info |= found->second | CI_HAS_BROAD;
            }
            const bool tie_within = mem.size() > 1 && (key_of[mem[1]] >> KEY_TUPLE_SHIFT) == (key_of[mem[0]] >> KEY_TUPLE_SHIFT);
            rec[CR_INFO] = info;
            rec[CR_GROUP] = group_mask;
            // Leaves of at most 16 classes keep the best member's output-predicate field mask above the group bits.
            if (order.size() <= 16) rec[CR_GROUP] |= r2_mask_of(best.flags) & 0xFFFF0000u;
            rec[CR_FIRST_FLAGS] = flags_of(mem[0]);
            {
                // Flags whose rule cannot fire while this class is the top candidate are recorded as if its best
                // member carried them: the kernel then never takes them for "carried by some candidate but not by
                // the top one".  A rule cannot fire when the bits this class demands of a word contradict its
                // condition, or when it needs a property the best member lacks.
                const u128 m = best.weakest(), b = best.b_ok ? best.bbase : best.sbase;
                auto one = [&](int bit) { return ((m >> bit) & 1) && ((b >> bit) & 1); };
                auto zero = [&](int bit) { return ((m >> bit) & 1) && !((b >> bit) & 1); };
                uint32_t off = 0;
                if (one(87) && one(88) && one(89)) off |= FL_HAS_TP | FL_LEA_A1 | FL_LEA_A2;
                if (one(81) && one(82) && one(83)) off |= FL_HAS_OUTPRED_F | FL_LEA_A1;
                if (zero(81) || zero(82) || zero(83)) off |= FL_NO_MID_P | FL_LEA_A2;
                for (int bit = 64; bit < 72; ++bit)
                    if (zero(bit)) off |= FL_SHL_OK;
                if (!(best.flags & FL1_HAS_R2)) off |= FL_NO_OUTPRED;
                if (!(best.flags & FL1_IS_LEA)) off |= FL_LEA_A1 | FL_LEA_A2;
                if (!(best.flags & FL1_IS_ULOP3)) off |= FL_ENDS_UP;
                if (one(32) || one(33)) off |= FL_BRA_NOMODE;
                if (zero(32) || one(33)) off |= FL_EXP_U | FL_GRP_U;
                if (one(32) || zero(33)) off |= FL_EXP_DIV | FL_GRP_DIV;
                if (zero(32) || zero(33)) off |= FL_EXP_CONV | FL_GRP_CONV;
                rec[CR_FIRST_FLAGS] |= off & ~strip;
            }
            rec[CR_KEY] = key_of[mem[0]] | (tie_within ? (uint32_t)KEY_WITHIN : 0u);
            rec[CR_BEST] = mem[0] | (ext_of[mem[0]] << 16);
            uint32_t any = 0;
            for (uint32_t v : mem) any |= flags_of(v) & 0xFFFFu;
            if (mem.size() > 1) {
                // Best member per choice flag (members are in rank order) and whether it is tied.
                // The per-flag tables are indexed by the class itself (classes with one member leave a gap),
                // so the kernel finds one without reading the class's cold quad first.
                ft.flagbest.resize((size_t(first_class) + ci) * FB_WORDS, 0);
                rec[CR_FLAGBEST] = uint32_t(ft.flagbest.size() / FB_WORDS);
                uint32_t fb[FB_WORDS] = {0};
                for (int f = 0; f < 16; ++f) {
                    int seen = 0;
                    uint32_t first_key = 0;
                    for (uint32_t v : mem) {
                        if (!((flags_of(v) >> f) & 1u)) continue;
                        if (seen == 0) { first_key = key_of[v]; fb[2 * f] = key_of[v]; fb[2 * f + 1] = v | (ext_of[v] << 16); }
                        else if (seen == 1 && (key_of[v] >> KEY_TUPLE_SHIFT) == (first_key >> KEY_TUPLE_SHIFT)) fb[2 * f] |= KEY_WITHIN;
                        ++seen;
                    }
                }
                ft.flagbest.insert(ft.flagbest.end(), fb, fb + FB_WORDS);
            }
            rec[CR_ANY_FLAGS] = any;
            rec[CR_SMASK] |= any;   // the test reads the flags from here
            if (ci < 16 && (info & CI_HAS_BROAD)) leaf_broad16 |= 1u << ci;
            if (info & CI_HAS_BROAD) leaf_has_broad = true;
            ft.classes.insert(ft.classes.end(), rec, rec + CR_WORDS);
            leaf_group[ci] = group_mask; leaf_key[ci] = rec[CR_KEY] & ~(uint32_t)KEY_WITHIN; leaf_within[ci] = tie_within ? 1u : 0u;
        }
        // Broad records that cannot change the outcome once class k is the first strict match of the leaf: k has
        // a non-negative score (so a strict match is on top whatever else matches: k itself or a later class of
        // its group), and the broad class's choice flags are carried, or ruled out, by each of those possible
        // top candidates (so its flags add nothing to what the rules look at, and the second pass, which asks
        // for a flag the top candidate lacks, would pass it over).  The rest are the ones that still matter:
        // one word per class, kept in the upper half of its info word.
        const size_t n16 = std::min<size_t>(order.size(), 16);
        std::vector<uint32_t> relevant(order.size(), 0);
        uint32_t leaf_relevant = 0;
        for (size_t k = 0; k < n16; ++k) {
            const uint32_t* rk = &ft.classes[(size_t(first_class) + k) * CR_WORDS];
            if (!st[groups[order[k]][0]].s_ok) continue;
            uint32_t common = rk[CR_FIRST_FLAGS] & 0xFFFFu;
            bool nonneg = !(rk[CR_KEY] >> 31);
            if (order.size() <= 16) {
                for (size_t j = k + 1; j < n16; ++j)
                    if ((rk[CR_GROUP] >> j) & 1u) common &= ft.classes[(size_t(first_class) + j) * CR_WORDS + CR_FIRST_FLAGS];
            } else {
                // Leaves beyond 16 classes are ranked 32 at a time by a path of its own: one answer for the whole leaf.
                for (size_t j = 0; j < order.size(); ++j) {
                    const uint32_t* rj = &ft.classes[(size_t(first_class) + j) * CR_WORDS];
                    if (!st[groups[order[j]][0]].s_ok) continue;
                    common &= rj[CR_FIRST_FLAGS];
                    if (rj[CR_KEY] >> 31) nonneg = false;
                }
            }
            for (size_t j = 0; j < n16; ++j) {
                const uint32_t* rj = &ft.classes[(size_t(first_class) + j) * CR_WORDS];
                if ((rj[CR_INFO] & CI_HAS_BROAD) && (!nonneg || (rj[CR_ANY_FLAGS] & 0xFFFFu & ~common))) relevant[k] |= 1u << j;
            }
            leaf_relevant |= relevant[k];
        }
        // How far the kernel has to test the leaf's classes once class f is the first strict match: up to the
        // last class that can still change the outcome — a later class of f's group (it could outrank or tie f),
        // a later class with a broad record that matters beside f (it has to be tested strictly before it is
        // tested broadly), or a later class that carries a flag some rule could ask for: a flag that f, a later
        // class that can match together with f, or one of f's own members carries and that some possible top
        // candidate (f or a later class of its group) neither carries nor rules out.  Class i records, one bit
        // per first match f <= i, whether the walk may end after it (bits 15:0 of its first base word, which the
        // match test leaves out).
        if (order.size() <= 16) {
            std::vector<size_t> last(order.size());
            for (size_t f = 0; f < order.size(); ++f) {
                const uint32_t* rf = &ft.classes[(size_t(first_class) + f) * CR_WORDS];
                last[f] = order.size() - 1;
                if (!st[groups[order[f]][0]].s_ok) continue;   // never a strict match
                const uint32_t later = ~((2u << f) - 1u) & 0xFFFFu;
                const uint32_t rivals = rf[CR_GROUP] & later;
                uint32_t common = rf[CR_FIRST_FLAGS] & 0xFFFFu, carried = rf[CR_ANY_FLAGS] & 0xFFFFu;
                for (size_t c = f + 1; c < order.size(); ++c) {
                    const uint32_t* rc = &ft.classes[(size_t(first_class) + c) * CR_WORDS];
                    if ((rivals >> c) & 1u) common &= rc[CR_FIRST_FLAGS];
                    if (can_both_match(order[f], order[c])) carried |= rc[CR_ANY_FLAGS] & 0xFFFFu;
                }
                const uint32_t asked = carried & ~common;
                uint32_t needed = rivals | (relevant[f] & later);
                for (size_t c = f + 1; c < order.size(); ++c)
                    if (can_both_match(order[f], order[c]) && (ft.classes[(size_t(first_class) + c) * CR_WORDS + CR_ANY_FLAGS] & asked))
                        needed |= 1u << c;
                last[f] = f;
                for (size_t c = f + 1; c < order.size(); ++c)
                    if ((needed >> c) & 1u) last[f] = c;
            }
            for (size_t i = 0; i < order.size(); ++i) {
                uint32_t done = 0;
                for (size_t f = 0; f <= i; ++f)
                    if (last[f] <= i) done |= 1u << f;
                ft.classes[(size_t(first_class) + i) * CR_WORDS + CR_SBASE] |= done;
            }
        }
        // The second pass asks for the best member that carries one flag among the matching classes.  When exactly
        // one class of the leaf carries the flag at all, the answer does not depend on the word.
        if (order.size() <= 16) {
            ft.leafbest.resize((size_t(first_class) + 1) * FB_WORDS, 0);
            uint32_t* lb = &ft.leafbest[size_t(first_class) * FB_WORDS];
            for (uint32_t f = 0; f < 16; ++f) {
                size_t carrier = order.size(), carriers = 0;
                for (size_t c = 0; c < order.size(); ++c)
                    if ((ft.classes[(size_t(first_class) + c) * CR_WORDS + CR_ANY_FLAGS] >> f) & 1u) { carrier = c; ++carriers; }
                if (carriers != 1) continue;
                const uint32_t* rc = &ft.classes[(size_t(first_class) + carrier) * CR_WORDS];
                if (rc[CR_INFO] & CI_SEVERAL) {
                    const uint32_t* fb = &ft.flagbest[size_t(rc[CR_FLAGBEST]) * FB_WORDS];
                    lb[2 * f] = 1u | ((fb[2 * f] & KEY_WITHIN) ? 2u : 0u);
                    lb[2 * f + 1] = fb[2 * f + 1];
                } else {
                    lb[2 * f] = 1u;
                    lb[2 * f + 1] = rc[CR_BEST];
                }
            }
        }
        // Words of the whole leaf ride in the upper halves of the flag words.
        for (size_t ci = 0; ci < n16; ++ci)
            ft.classes[(size_t(first_class) + ci) * CR_WORDS + CR_INFO] |= relevant[ci] << CI_LEAF_POS;
        ft.classes[size_t(first_class) * CR_WORDS + CR_ANY_FLAGS] |= leaf_broad16 << CI_LEAF_POS;
        ft.n_leaves++;
        ft.max_leaf_classes = std::max<uint32_t>(ft.max_leaf_classes, uint32_t(order.size()));
        return REF_LEAF | first_class | (uint32_t(order.size()) << 20) | (leaf_has_broad ? uint32_t(REF_BROAD) : 0u) |
               (leaf_relevant ? uint32_t(REF_BROAD_ALWAYS) : 0u);
    }

    // The node hash before its final shift: one multiplier per limb, summed (three multiply-adds
    // on the device).
    static uint32_t mix(u128 x, const uint32_t m[3]) {
        return uint32_t(x) * m[0] + uint32_t(x >> 32) * m[1] + uint32_t(x >> 64) * m[2];
    }
    // Fills node record `node` and returns the ref to it.
    uint32_t write_node(uint32_t node, u128 mask, const uint32_t m[3], uint32_t child_base, uint32_t shift) {
        uint32_t* n = &ft.nodes[size_t(node) * NR_WORDS];
        n[NR_MASK0] = uint32_t(mask); n[NR_MASK1] = uint32_t(mask >> 32); n[NR_MASK2] = uint32_t(mask >> 64);
        n[NR_MULT0] = m[0]; n[NR_MULT1] = m[1]; n[NR_MULT2] = m[2];
        n[NR_CHILD] = child_base;
        n[NR_SHIFT] = shift;
        return REF_NODE | node | ((n[NR_MASK0] | n[NR_MASK1]) ? uint32_t(REF_WIDE) : 0u);
    }
    static void draw_multipliers(uint64_t* rng, uint32_t m[3]) {
        for (int k = 0; k < 3; ++k) { *rng = splitmix64(*rng); m[k] = uint32_t(*rng >> 16) | 1u; }
    }

    // A subtree of bit nodes becomes one hash node over its bits (at most kFlattenBits of them;
    // deeper parts become hash nodes of their own): one step instead of a chain, and the kernel
    // walks nodes of one kind only.  Every assignment of the bits is walked through the bit
    // nodes here, so the new node reaches exactly the refs the chain reached.
    static constexpr uint32_t kFlattenBits = 7;
    static constexpr size_t kBitParts = 32;       // hash levels of at most this many parts are split bit by bit instead
    static constexpr size_t kLeafUnderHash = 4;   // at most this many classes directly under a hash node are not split further
    uint32_t flatten_bits(uint32_t root) {
        if (!(root & REF_BIT)) return root;
        // Fewer bits when no multiplier separates all assignments of the full set (one bit always works).
        for (uint32_t max_bits = kFlattenBits; max_bits >= 1; --max_bits) {
            const uint32_t r = flatten_bits(root, max_bits);
            if (r) return r;
        }
        throw std::runtime_error("no perfect hash for a bit-node subtree");
    }
    uint32_t flatten_bits(uint32_t root, uint32_t max_bits) {
        std::vector<uint32_t> bits;
        {
            std::vector<uint32_t> queue{root};
            for (size_t q = 0; q < queue.size(); ++q) {
                const uint32_t r = queue[q];
                if (!(r & REF_BIT) || (r & REF_LEAF)) continue;
                const uint32_t bit = (r >> 20) & 127u;
                if (std::find(bits.begin(), bits.end(), bit) == bits.end()) {
                    if (bits.size() >= max_bits) continue;
                    bits.push_back(bit);
                }
                queue.push_back(ft.children[ref_index(r)]);
                queue.push_back(ft.children[ref_index(r) + 1]);
            }
        }
        const uint32_t k = uint32_t(bits.size());
        std::vector<u128> pattern(size_t(1) << k);
        std::vector<uint32_t> target(size_t(1) << k);
        u128 mask = 0;
        for (uint32_t b : bits) mask |= (u128)1 << b;
        for (uint32_t a = 0; a < (1u << k); ++a) {
            u128 x = 0;
            for (uint32_t j = 0; j < k; ++j)
                if ((a >> j) & 1u) x |= (u128)1 << bits[j];
            uint32_t r = root;
            while ((r & REF_BIT) && !(r & REF_LEAF)) {
                const uint32_t bit = (r >> 20) & 127u;
                if (std::find(bits.begin(), bits.end(), bit) == bits.end()) break;
                r = ft.children[ref_index(r) + uint32_t((x >> bit) & 1)];
            }
            pattern[a] = x;
            target[a] = r;
        }
        uint64_t rng = 0x13198A2E03707344ull ^ root;
        for (uint32_t extra = 0; extra < 4; ++extra) {
            const uint32_t kk = k + extra;
            for (uint32_t attempt = 0; attempt < 4000; ++attempt) {
                uint32_t m[3];
                draw_multipliers(&rng, m);
                std::vector<char> seen(size_t(1) << kk, 0);
                bool clash = false;
                for (const u128& x : pattern) {
                    const uint32_t h = kk ? mix(x, m) >> (32 - kk) : 0u;
                    if (seen[h]) { clash = true; break; }
                    seen[h] = 1;
                }
                if (clash) continue;
                const uint32_t node = uint32_t(ft.nodes.size() / NR_WORDS);
                ft.nodes.resize(ft.nodes.size() + NR_WORDS, 0);
                const uint32_t child_base = uint32_t(ft.children.size());
                if (child_base + (size_t(1) << kk) >= (1u << 20)) throw std::runtime_error("match tree too large");
                ft.children.resize(ft.children.size() + (size_t(1) << kk), REF_LEAF);
                for (size_t i = 0; i < pattern.size(); ++i)
                    ft.children[child_base + (kk ? mix(pattern[i], m) >> (32 - kk) : 0u)] = target[i];
                return write_node(node, mask, m, child_base, 32 - kk);
            }
        }
        return 0;
    }
    // Replaces every bit node reachable from `dir` (entries added on the way are visited too).
    void flatten_all(std::vector<uint32_t>& dir) {
        for (uint32_t& r : dir) r = flatten_bits(r);
        for (size_t i = 0; i < ft.children.size(); ++i) {
            const uint32_t r = ft.children[i];
            if ((r & REF_BIT) && !(r & REF_LEAF) && reachable_as_child_of_node(i)) {
                const uint32_t nr = flatten_bits(r);
                ft.children[i] = nr;
            }
        }
    }
    // Child-table entries of hash nodes are the only ones the walk can still reach; entries of
    // the two-entry tables of replaced bit nodes are dead.
    bool reachable_as_child_of_node(size_t index) const {
        for (size_t n = 0; n * NR_WORDS < ft.nodes.size(); ++n) {
            const uint32_t base = ft.nodes[n * NR_WORDS + NR_CHILD], size = uint32_t(1) << (32 - ft.nodes[n * NR_WORDS + NR_SHIFT]);
            if (index >= base && index < size_t(base) + size) return true;
        }
        return false;
    }

    // Splits `vs` on the mask bits that all of them check (beyond `used`), then on single
    // bits that most of them check; recursion ends in leaves that no bit shrinks further.
    uint32_t build(const std::vector<uint32_t>& vs, u128 used, uint32_t depth, bool under_hash = false) {
        max_depth = std::max(max_depth, depth);
        // Directly under a hash node a further split costs every word that passes a step of its own (bit nodes
        // under bit nodes are folded into one step, hash nodes are not): a handful of classes stays a leaf there.
        if (under_hash && class_count(vs) <= kLeafUnderHash) return make_leaf(vs);
        u128 common = (((u128)1) << 96) - 1;
        for (uint32_t v : vs) common &= st[v].weakest();
        common &= ~used;
        std::map<u128, std::vector<uint32_t>> parts;
        if (vs.size() > 1 && common)
            for (uint32_t v : vs) parts[st[v].base96 & common].push_back(v);
        if (parts.size() > 1 && parts.size() <= kBitParts) {
            // A few parts: split them on one of the common bits, the most even one.  Chains of such bit nodes (and
            // of the single-bit splits below) are folded into one hash node later, so that several small levels
            // cost one step: the SM120 table walks 0.9 steps per word and 1.1 per warp this way, against 1.1 and
            // 2.3 with a hash node per level.
            int best_bit = -1;
            size_t best_max = parts.size();
            for (int bit = 12; bit < 96; ++bit) {
                if (!((common >> bit) & 1)) continue;
                size_t ones = 0;
                for (const auto& kv : parts) ones += size_t((kv.first >> bit) & 1);
                const size_t mx = std::max(ones, parts.size() - ones);
                if (mx < best_max) { best_max = mx; best_bit = bit; }
            }
            if (best_bit >= 0) {
                std::vector<uint32_t> zero, one;
                for (uint32_t v : vs) (((st[v].base96 >> best_bit) & 1) ? one : zero).push_back(v);
                const uint32_t child_base = uint32_t(ft.children.size());
                if (child_base + 2 >= (1u << 20)) throw std::runtime_error("match tree too large");
                ft.children.resize(ft.children.size() + 2, REF_LEAF);
                const u128 m = ((u128)1) << best_bit;
                const uint32_t z = build(zero, used | m, depth + 1);
                const uint32_t o = build(one, used | m, depth + 1);
                ft.children[child_base] = z;
                ft.children[child_base + 1] = o;
                return REF_BIT | child_base | (uint32_t(best_bit) << 20);
            }
        }
        if (parts.size() > 1) {
            // Perfect hash of the masked word into a power-of-two child table.
            uint32_t bits = 1;
            while ((1u << bits) < parts.size()) ++bits;
            uint32_t mult[3] = {0, 0, 0};
            bool ok = false;
            uint64_t rng = 0x243F6A8885A308D3ull ^ (uint64_t(vs[0]) << 20) ^ depth;
            for (uint32_t extra = 0; extra < 3 && !ok; ++extra) {
                const uint32_t k = bits + extra;
                for (uint32_t attempt = 0; attempt < 4000 && !ok; ++attempt) {
                    uint32_t m[3];
                    draw_multipliers(&rng, m);
                    std::vector<char> seen(size_t(1) << k, 0);
                    bool clash = false;
                    for (const auto& kv : parts) {
                        const uint32_t h = mix(kv.first, m) >> (32 - k);
                        if (seen[h]) { clash = true; break; }
                        seen[h] = 1;
                    }
                    if (!clash) { ok = true; mult[0] = m[0]; mult[1] = m[1]; mult[2] = m[2]; bits = k; }
                }
            }
            if (ok) {
                const uint32_t node = uint32_t(ft.nodes.size() / NR_WORDS);
                ft.nodes.resize(ft.nodes.size() + NR_WORDS, 0);
                const uint32_t child_base = uint32_t(ft.children.size());
                ft.children.resize(ft.children.size() + (size_t(1) << bits), REF_LEAF);   // empty leaf: nothing matches
                for (const auto& kv : parts) {
                    const uint32_t h = mix(kv.first, mult) >> (32 - bits);
                    const uint32_t ref = build(kv.second, used | common, depth + 1, true);
                    ft.children[child_base + h] = ref;
                }
                return write_node(node, common, mult, child_base, 32 - bits);
            }
            // No perfect hash found: fall through and scan (still correct).
        }

        // Single-bit split: candidates that do not check the bit go to both sides.
        const size_t n_classes = class_count(vs);
        // A leaf above 128 candidates may not fit the 32-bit rank keys: split it whatever the cost.
        const bool oversize = vs.size() > 128;
        if (n_classes > 2) {
            size_t best_max = n_classes, best_sum = 0;
            int best_bit = -1;
            std::vector<uint32_t> best_zero, best_one;
            for (int bit = 12; bit < 96; ++bit) {
                const u128 m = ((u128)1) << bit;
                if (used & m) continue;
                std::vector<uint32_t> zero, one;
                for (uint32_t v : vs) {
                    const bool checks = (st[v].weakest() & m) != 0, set = (st[v].base96 & m) != 0;
                    if (!checks || !set) zero.push_back(v);
                    if (!checks || set) one.push_back(v);
                }
                if (zero.size() == vs.size() && one.size() == vs.size()) continue;
                const size_t cz = class_count(zero), co = class_count(one);
                const size_t mx = std::max(cz, co), sum = cz + co;
                // Candidates that do not check the bit are copied to both sides: bound that growth.
                if (sum > 2 * n_classes && !oversize) continue;
                if (mx < best_max || (mx == best_max && best_bit >= 0 && sum < best_sum)) {
                    best_max = mx; best_sum = sum; best_bit = bit; best_zero = zero; best_one = one;
                }
            }
            if (best_bit >= 0 && best_max < n_classes && (oversize || ft.classes.size() / CR_WORDS < class_budget)) {
                const uint32_t child_base = uint32_t(ft.children.size());
                if (child_base + 2 >= (1u << 20)) throw std::runtime_error("match tree too large");
                ft.children.resize(ft.children.size() + 2, REF_LEAF);
                const u128 m = ((u128)1) << best_bit;
                const uint32_t z = best_zero.empty() ? uint32_t(REF_LEAF) : build(best_zero, used | m, depth + 1);
                const uint32_t o = best_one.empty() ? uint32_t(REF_LEAF) : build(best_one, used | m, depth + 1);
                ft.children[child_base] = z;
                ft.children[child_base + 1] = o;
                return REF_BIT | child_base | (uint32_t(best_bit) << 20);
            }
        }
        return make_leaf(vs);
    }
};

}  // namespace

FlatTable FlatTable::compile(const IsaTable& t) {
    const size_t nv = t.variants.size();
    if (nv >= 0xFFFF) throw std::runtime_error("table has too many variants for a u16 form id");
    FlatTable ft;
    ft.n_keys = uint32_t(t.keys.size());
    ft.meta.resize(nv);
    ft.var.assign(nv * VR_WORDS, 0);
    ft.gindex.assign(nv, 0);
    ft.ext.assign(nv * XR_WORDS, 0);

    const u128 kGuard = 0xF000;
    const u128 kLow96 = (((u128)1) << 96) - 1;
    const u128 kStdRegs = ((u128)0xFF << 16) | ((u128)0xFF << 24) | ((u128)0xFFFFFFFFull << 32) | ((u128)0xFF << 64);
    std::vector<Static> st(nv);
    std::map<std::array<uint32_t, 4>, uint32_t> rt_mask_index;

    for (size_t vi = 0; vi < nv; ++vi) {
        const IsaVariant& v = t.variants[vi];
        const std::string& key = t.keys[v.key_id].name;
        const IsaKey& ik = t.keys[v.key_id];
        Static& s = st[vi];
        VariantMeta& m = ft.meta[vi];
        m.key = key; m.mod_group = v.mod_group; m.key_id = v.key_id; m.opcode = opcode_of(key);

        // Match masks (reference src/decoder.rs:93-145).  The "relaxed" mask of the reference
        // removes immediate-like field ranges from a mask that already excludes every field
        // range, so it always equals the strict mask; the compile checks that and drops it.
        u128 field_mask = 0, imm_mask = 0;
        bool any_opaque = false;
        for (const IsaField& f : v.fields) {
            field_mask |= f.range();
            switch (f.ext) {
                case Ext::Imm: case Ext::ImmShr: case Ext::ImmDec: case Ext::ImmDecU32: case Ext::F32: case Ext::F16:
                case Ext::F16d: case Ext::F64hi: case Ext::SubR: case Ext::SubUR: case Ext::SubImm: case Ext::SubImmS24:
                case Ext::SubRShr: case Ext::SubURShr: case Ext::SubImmShr: imm_mask |= f.range(); break;
                default: break;
            }
            if (f.ext == Ext::OpaqueModifier) any_opaque = true;
        }
        const u128 match = ~v.variable_mask & ~field_mask;
        const u128 relaxed = match & ~imm_mask;
        if (relaxed != match) throw std::runtime_error("internal: relaxed mask differs from strict mask for " + key);
        const u128 broad = relaxed & ~kStdRegs;
        const bool broad_eligible = v.fields.empty() || contains(key, "_ARI") || contains(key, "_AI") ||
                                    contains(key, "dARI") || contains(key, "ARURI");
        // The word is matched with bits 127:96 cleared, so a mask that demands a one up there
        // can never match.
        const u128 sm = match & ~kGuard, bm = broad & ~kGuard;
        s.s_ok = ((v.and_base & sm) >> 96) == 0;
        s.b_ok = broad_eligible && ((v.and_base & bm) >> 96) == 0;
        s.smask = sm & kLow96; s.sbase = v.and_base & sm & kLow96;
        s.bmask = bm & kLow96; s.bbase = v.and_base & bm & kLow96;
        s.base96 = v.and_base & kLow96;

        // Static rank components (reference src/decoder.rs:213-279).
        s.score = consistency_score(key, v);
        m.score = s.score;
        const bool global_mem = starts_with(key, "LDG") || starts_with(key, "STG") || starts_with(key, "LDGSTS") ||
                                starts_with(key, "ATOMG") || starts_with(key, "REDG");
        int plain_addr = 0;
        if (global_mem && !contains(key, "dARI") && !contains(key, "dAI") && (contains(key, "_ARI") || contains(key, "_AI")))
            plain_addr = 1;
        int undiscovered = 0;
        if (ends_with(key, "_?") || contains(key, "_?_") || contains(key, "_II_?")) undiscovered = 50;
        else if (contains(key, "_II_II_UR") || contains(key, "_II_UR") || contains(key, "_UR_II") ||
                 contains(key, "_II_II_?") || contains(key, "_R_II_?") || contains(key, "_P_II_II"))
            undiscovered = 30;
        const int adj_len = int(key.size()) - (s.score >= 3 ? 10 : 0);
        s.mid = std::make_tuple(any_opaque ? 1 : 0, plain_addr, undiscovered, adj_len, -s.score);
        s.lo = std::make_tuple(-popcount128(match), -int(v.mod_group.size()));

        // Rule flags (reference src/decoder.rs:391-599).
        const std::vector<std::string> types = operand_types(key);
        bool has_mid_p = false;
        if (types.size() > 2)
            for (size_t i = 1; i + 1 < types.size(); ++i) has_mid_p |= is_pred_type(types[i]);
        bool key_has_pred = false;
        for (size_t i = 1; i < types.size(); ++i) key_has_pred |= is_pred_type(types[i]);
        bool field_pred_tok = false, has_tp = false, has_outpred_f = false;
        int r2_shift = -1, r2_bits = 0;
        for (const IsaField& f : v.fields) {
            if (f.ext != Ext::Pred) continue;
            if (f.token_idx >= 1) field_pred_tok = true;
            if (f.shift >= 87) has_tp = true;
            if (f.token_idx >= 1 && f.token_idx <= 3 && f.shift >= 80 && f.shift <= 85) {
                has_outpred_f = true;
                if (r2_shift < 0) { r2_shift = int(f.shift); r2_bits = int(f.bits); }
            }
        }
        const bool ends_p = ends_with(key, "_P") || ends_with(key, "_UP");
        uint32_t fl = 0;
        if (starts_with(key, "BRA")) fl |= FL_IS_BRA;
        static const char* kModes[3] = {"U", "DIV", "CONV"};
        bool any_mode = false;
        for (int k = 0; k < 3; ++k) {
            if (names_mode_in_opcode(key, kModes[k])) { fl |= FL_EXP_U << k; any_mode = true; }
            if (names_mode_in_group(v.mod_group, kModes[k])) { fl |= FL_GRP_U << k; any_mode = true; }
        }
        if (!any_mode) fl |= FL_BRA_NOMODE;
        if (!(key_has_pred || field_pred_tok)) fl |= FL_NO_OUTPRED;
        if (s.score >= 0 && contains(v.mod_group, "SHL")) fl |= FL_SHL_OK;
        if (ends_p && has_tp) fl |= FL_LEA_A1;
        if (ends_p && has_tp && !has_mid_p) fl |= FL_LEA_A2;
        if (has_tp) fl |= FL_HAS_TP;
        if (ends_with(key, "_UP")) fl |= FL_ENDS_UP;
        if (has_outpred_f) fl |= FL_HAS_OUTPRED_F;
        if (!has_mid_p) fl |= FL_NO_MID_P;
        if (starts_with(key, "LEA_") || starts_with(key, "ULEA_")) fl |= FL1_IS_LEA;
        if (starts_with(key, "ULOP3") || starts_with(key, "UPLOP3")) fl |= FL1_IS_ULOP3;
        // The rule compares that field with all ones; a field reaching past bit 95 reads zeros there
        // (the word is matched with bits 127:96 cleared) and can never be all ones.
        if (r2_shift >= 0 && r2_shift + r2_bits <= 96) {
            fl |= FL1_HAS_R2 | (uint32_t(r2_shift - 80) << FL1_R2_SHIFT_POS) | (uint32_t(r2_bits - 1) << FL1_R2_BITS_POS);
        }
        s.flags = fl;

        // ---- slot layout ---------------------------------------------------------------------
        // Only field bits below bit 96 are stored.  Layout 0: every multi-bit field has a slot of
        // its own, chosen by the limb it lies in — limb 0 fields take slots 0, 1, 2; the first
        // limb 1 field slot 3, further ones slots 5, 6; the first limb 2 field slot 4, further
        // ones slots 6, 5 (each in table order) — and the 1-bit fields share slot 7 at
        // (source bit mod 32) rotated by a per-limb amount so that the three limbs do not
        // collide.  Layout 1 (when a field crosses a limb boundary, the fields do not fit that
        // pattern, or stored field ranges overlap): bits stay in place, slot k = limb k.
        auto stored_bits = [](const IsaField& f) -> uint32_t {
            return f.shift >= 96 ? 0u : std::min<uint32_t>(f.shift + f.bits, 96) - f.shift;
        };
        u128 stored_union = 0;
        bool overlap = false, crossing = false;
        uint32_t per_limb[3] = {0, 0, 0};
        uint32_t fm[3] = {0, 0, 0};
        bool dup_flag = false;
        for (const IsaField& f : v.fields) {
            const uint32_t sb = stored_bits(f);
            if (!sb) continue;
            const u128 r = ((((u128)1) << sb) - 1) << f.shift;
            if (stored_union & r) overlap = true;
            stored_union |= r;
            if (sb == 1) {
                if (fm[f.shift >> 5] & (1u << (f.shift & 31))) dup_flag = true;
                fm[f.shift >> 5] |= 1u << (f.shift & 31);
            } else if ((f.shift >> 5) != ((f.shift + sb - 1) >> 5)) {
                crossing = true;
            } else {
                ++per_limb[f.shift >> 5];
            }
        }
        const bool has_flags = (fm[0] | fm[1] | fm[2]) != 0;
        uint32_t rot1 = 0, rot2 = 0;
        bool rot_ok = !has_flags;
        for (uint32_t a = 0; a < 32 && !rot_ok; ++a)
            for (uint32_t b = 0; b < 32 && !rot_ok; ++b) {
                const uint32_t x = fm[0], y = cb_rotl(fm[1], a), z = cb_rotl(fm[2], b);
                if (!(x & y) && !(x & z) && !(y & z)) { rot_ok = true; rot1 = a; rot2 = b; }
            }
        const uint32_t extra1 = per_limb[1] > 1 ? per_limb[1] - 1 : 0, extra2 = per_limb[2] > 1 ? per_limb[2] - 1 : 0;
        const bool fits = per_limb[0] <= 3 && extra1 + extra2 <= 2;
        const bool layout0 = !overlap && !dup_flag && !crossing && rot_ok && fits;
        m.layout_kind = layout0 ? 0 : 1;
        uint32_t* xr = &ft.ext[vi * XR_WORDS];
        // Slots of the fields of limb 0, 1, 2 in the order they are handed out, and the multiplier
        // word (XR_MULT + ...) that serves each (slot, limb) pair.
        static const uint32_t kSlots[3][3] = {{0, 1, 2}, {3, 5, 6}, {4, 6, 5}};
        uint32_t limb2_slots = 0;   // slots 5 / 6 taken by a limb 2 field
        uint32_t taken[3] = {0, 0, 0};
        uint32_t amounts[7] = {0, 0, 0, 0, 0, 0, 0};
        const uint32_t gfield_start = uint32_t(ft.gfields.size());
        for (const IsaField& f : v.fields) {
            const uint32_t sb = stored_bits(f);
            uint32_t pos = 0xFFFFFFFFu;
            if (sb) {
                if (!layout0) pos = f.shift;
                else if (sb == 1) {
                    const uint32_t limb = f.shift >> 5, bit = f.shift & 31, r = limb == 0 ? 0 : (limb == 1 ? rot1 : rot2);
                    pos = 7 * 32 + ((bit + r) & 31);
                } else {
                    const uint32_t limb = f.shift >> 5, k = taken[limb]++;
                    const uint32_t slot = kSlots[limb][k];
                    pos = slot * 32;
                    xr[XR_MULT + slot] = 1u << (32u - (f.shift & 31u) - sb);
                    amounts[slot] = 32u - sb;
                    if (limb == 2 && slot == 5) limb2_slots |= XC_SLOT5_LIMB2;
                    if (limb == 2 && slot == 6) limb2_slots |= XC_SLOT6_LIMB2;
                }
            }
            FieldMeta fmeta;
            fmeta.shift = f.shift; fmeta.bits = f.bits; fmeta.token_idx = f.token_idx; fmeta.dst_pos = pos;
            fmeta.stored_bits = sb;
            fmeta.name = field_display_name(f); fmeta.extraction = f.ext_name;
            m.fields.push_back(fmeta);
            ft.gfields.push_back(f.shift | (f.bits << 7) | (gen_class(f) << 14) | ((sb ? pos : uint32_t(GF_NOT_STORED)) << 16));
        }
        for (uint32_t s = 0; s < 6; ++s) xr[XR_AMOUNT] |= amounts[s] << (5 * s);
        const uint32_t gfield_count = uint32_t(ft.gfields.size()) - gfield_start;
        if (gfield_count > 255 || ft.gfields.size() >= (1u << 24)) throw std::runtime_error("too many fields in " + key);
        if (layout0) { xr[XR_MASK] = fm[0]; xr[XR_MASK + 1] = fm[1]; xr[XR_MASK + 2] = fm[2]; }
        else for (int k = 0; k < 3; ++k) xr[XR_MASK + k] = uint32_t(stored_union >> (32 * k));

        // Synthesized abs/neg modifiers (reference src/decoder.rs:312-345).
        static const char* kNotAlu[] = {"LDG", "LDL", "LDS", "LDC", "LDCU", "STG", "STL", "STS", "ATOM", "RED", "BRA",
                                        "BSSY", "BSYNC", "EXIT", "RET", "BAR", "S2R", "S2UR", "LDSM", "LDGSTS", "QMMA"};
        const std::string base_op = base_op_of(key);
        bool is_alu = true;
        for (const char* n : kNotAlu) is_alu &= base_op != n;
        uint32_t synth = 0;
        if (is_alu) {
            static const int kBits[4] = {63, 62, 72, 73};
            for (int k = 0; k < 4; ++k) {
                const int b = kBits[k];
                bool covered = false;
                for (const IsaField& f : v.fields) covered |= int(f.shift) <= b && b < int(f.shift + f.bits);
                if (!((v.and_base >> b) & 1) && !covered) synth |= 1u << k;
            }
        }
        m.synth_mask = synth;
        xr[XR_CFG] = amounts[6] | (rot1 << XC_ROT1_POS) | (rot2 << XC_ROT2_POS) | (uint32_t(m.layout_kind) << XC_LAYOUT_POS) |
                     limb2_slots | (synth << XC_SYNTH_POS);
        {
            std::vector<std::string> parts = split(key, '_');
            int skip = 0;
            for (size_t i = 1; i < parts.size() && is_pred_type(parts[i]); ++i) ++skip;
            m.ra_tok = skip + 2; m.rb_tok = skip + 3;
        }

        // Encode-side facts.
        auto is_ext = [](const IsaField& f, std::initializer_list<Ext> set) {
            for (Ext e : set) if (f.ext == e) return true;
            return false;
        };
        bool full_guard = false, lo3 = false, neg15 = false;
        for (const IsaField& f : v.fields) {
            if (f.shift <= 12 && f.shift + f.bits >= 16 && f.ext == Ext::Guard) full_guard = true;
            if (f.shift <= 14 && f.shift + f.bits >= 15 && is_ext(f, {Ext::Guard, Ext::GuardLo3})) lo3 = true;
            if (f.shift == 15 && f.bits == 1 && is_ext(f, {Ext::GuardNeg, Ext::Inv, Ext::Neg})) neg15 = true;
        }
        const bool guard_default = !(full_guard || (lo3 && neg15));
        std::string mnemonic = split(key, '_')[0];
        for (const std::string& mod : split(v.mod_group, ',')) mnemonic += "." + mod;
        const bool qmma_sp = base_op == "QMMA" && contains(mnemonic, ".SP");
        // Which of bits 124:122 end up holding reuse3 after the field loop and the slot rule
        // (reference src/encoder.rs:1155-1179): 0 zero, 1 one, 2 reuse3[i].
        uint32_t keep = 0, konst = 0;
        static const uint32_t kSlotShift[3] = {24, 32, 64};
        for (int i = 0; i < 3; ++i) {
            const uint32_t b = 122 + i;
            int state = ((v.and_base >> b) & 1) ? 1 : 0;
            for (const IsaField& f : v.fields) {
                if (!(f.shift <= b && b < f.shift + f.bits)) continue;
                state = (f.ext == Ext::Reuse && f.shift >= 122 && f.shift + f.bits <= 125) ? 2 : 0;
            }
            const IsaField* slot_field = nullptr;
            for (const IsaField& f : v.fields)
                if (f.shift == kSlotShift[i] && f.bits == 8 && is_ext(f, {Ext::Reg, Ext::UReg, Ext::URegFf, Ext::RegFf})) {
                    slot_field = &f;
                    break;
                }
            if (slot_field) {
                bool explicit_tok = false;
                for (const IsaField& f : v.fields) explicit_tok |= f.ext == Ext::Reuse && f.token_idx == slot_field->token_idx;
                if (!explicit_tok) state = 2;
            }
            if (state == 2) keep |= 1u << i;
            if (state == 1) konst |= 1u << i;
        }

        // Fields the kernel-metadata inference reads (reference src/main.rs:806-829): every "reg"
        // field, and for BSSY the "barrier" / "imm" fields.  Values are truncated to u32 there.
        {
            uint32_t entries[16] = {0};
            size_t ne = 0;
            for (const IsaField& f : v.fields) {
                const bool reg = f.ext == Ext::Reg, bar = m.opcode == "BSSY" && (f.ext == Ext::Barrier || f.ext == Ext::Imm);
                if ((!reg && !bar) || f.shift >= 96) continue;
                if (ne == 16) throw std::runtime_error("too many register fields in " + key);
                const uint32_t bits = std::min<uint32_t>(std::min<uint32_t>(f.bits, 32), 96 - f.shift);
                entries[ne++] = f.shift | (bits << 7) | (uint32_t(reg ? MF_KIND_REG : MF_KIND_BARRIER) << 13);
                // A register field and a barrier field are told apart by kind; a BSSY "reg" field counts as a register.
            }
            for (size_t k = 0; k < 16; ++k) {
                if (k % 2 == 0) ft.metaf.push_back(0);
                ft.metaf.back() |= entries[k] << (16 * (k & 1));
            }
        }

        uint32_t* vr = &ft.var[vi * VR_WORDS];
        const u128 cleared = v.and_base & ~stored_union;
        {
            // Constants of the fused roundtrip check: copied bits M = stored field bits, the
            // synthesized-modifier bits, the guard nibble when encode writes it, minus bit 80 when
            // encode clears it; constant ones A = the rest of and_base.
            static const int kSynthBit[4] = {63, 62, 72, 73};
            u128 copied = stored_union;
            for (int k = 0; k < 4; ++k)
                if ((synth >> k) & 1u) copied |= ((u128)1) << kSynthBit[k];
            const u128 guard_bits = guard_default ? (u128)0xF000 : (u128)0;
            const u128 sp_bit = qmma_sp ? (((u128)1) << 80) : (u128)0;
            const u128 M = (copied | guard_bits) & ~sp_bit & kLow96;
            const u128 A = cleared & ~guard_bits & ~sp_bit & kLow96;
            if (A & M) throw std::runtime_error("internal: constant and copied bits overlap in " + key);
            const uint32_t epoch = ik.has_epoch ? ik.epoch_upper32 : 0x000fc200u;
            const uint32_t e3 = ik.ctrl_kind == CTRL_NORMAL ? 0u : (epoch & ~0x03FFFE00u);
            // Mask quads are shared between variants; the index travels in the scheduling-field
            // bits of the E3 word, which the comparison leaves out.
            const std::array<uint32_t, 4> mq = {~limb(M, 0), ~limb(M, 1), ~limb(M, 2), keep | (konst << 3)};
            auto found = rt_mask_index.find(mq);
            if (found == rt_mask_index.end()) {
                found = rt_mask_index.emplace(mq, uint32_t(ft.rt_masks.size() / 4)).first;
                ft.rt_masks.insert(ft.rt_masks.end(), mq.begin(), mq.end());
            }
            if (found->second >= (1u << 17) || (e3 & 0x03FFFE00u)) throw std::runtime_error("internal: roundtrip mask index does not fit");
            for (int k = 0; k < 3; ++k) ft.rt.push_back(limb(A, k));
            ft.rt.push_back(e3 | (found->second << 9));
        }
        vr[VR_BASE] = limb(cleared, 0); vr[VR_BASE + 1] = limb(cleared, 1); vr[VR_BASE + 2] = limb(cleared, 2);
        vr[VR_EPOCH] = ik.has_epoch ? ik.epoch_upper32 : 0x000fc200u;
        ft.gindex[vi] = gfield_start | (gfield_count << 24);
        vr[VR_FLAGS] = (synth << VF_SYNTH_POS) | (keep << VF_REUSE_KEEP_POS) | (konst << VF_REUSE_CONST_POS) |
                       (guard_default ? VF_GUARD_DEFAULT : 0) | (qmma_sp ? VF_QMMA_SP : 0) |
                       (uint32_t(ik.ctrl_kind) << VF_CTRL_KIND_POS) | (m.opcode == "EXIT" ? VF_IS_EXIT : 0) |
                       (m.opcode == "BSSY" ? VF_IS_BSSY : 0);
    }

    // Variants with the same field layout share one extraction record.
    std::vector<uint32_t> ext_of(nv);
    {
        std::map<std::vector<uint32_t>, uint32_t> seen;
        std::vector<uint32_t> unique;
        for (size_t vi = 0; vi < nv; ++vi) {
            std::vector<uint32_t> rec(ft.ext.begin() + vi * XR_WORDS, ft.ext.begin() + (vi + 1) * XR_WORDS);
            auto it = seen.find(rec);
            if (it == seen.end()) {
                it = seen.emplace(rec, uint32_t(unique.size() / XR_WORDS)).first;
                unique.insert(unique.end(), rec.begin(), rec.end());
            }
            ext_of[vi] = it->second;
            ft.var[vi * VR_WORDS + VR_EXT] = it->second;
        }
        // The all-zero record (no field, no flag, no synthesized modifier): what a rejected word is extracted through.
        {
            const std::vector<uint32_t> zero(XR_WORDS, 0);
            auto it = seen.find(zero);
            if (it == seen.end()) {
                it = seen.emplace(zero, uint32_t(unique.size() / XR_WORDS)).first;
                unique.insert(unique.end(), zero.begin(), zero.end());
            }
            ft.at.zero_ext = it->second;
        }
        if (unique.size() / XR_WORDS > 0xFFFF) throw std::runtime_error("too many distinct field layouts");
        ft.ext.swap(unique);
    }
    // The encoder's deposit records, one per extraction record and derived from it alone.
    {
        const size_t n_ext = ft.ext.size() / XR_WORDS;
        ft.enc.assign(n_ext * ER_WORDS, 0);
        std::vector<uint32_t> rot_a(n_ext, 0), rot_b(n_ext, 0);
        for (size_t r = 0; r < n_ext; ++r) {
            const uint32_t* xr = &ft.ext[r * XR_WORDS];
            uint32_t* er = &ft.enc[r * ER_WORDS];
            const uint32_t cfg = xr[XR_CFG];
            uint32_t amount[8] = {0, 0, 0, 0, 0, 0, 0, 0}, amount7[3] = {0, 0, 0};
            if ((cfg >> XC_LAYOUT_POS) & 1u) {
                for (uint32_t k = 0; k < 3; ++k) er[ER_MASK + 3 * k + k] = xr[XR_MASK + k];   // slot k is limb k, in place
            } else {
                for (uint32_t s = 0; s < 7; ++s) {
                    const uint32_t mult = xr[XR_MULT + s];
                    if (!mult) continue;
                    const uint32_t limb = s < 3 ? 0u : (s == 3 ? 1u : (s == 4 ? 2u : ((cfg & (s == 5 ? XC_SLOT5_LIMB2 : XC_SLOT6_LIMB2)) ? 2u : 1u)));
                    const uint32_t right = ((s < 6 ? xr[XR_AMOUNT] >> (5 * s) : cfg) & 31u), take = 32u - right;
                    const uint32_t sh = 32u - take - uint32_t(__builtin_ctz(mult));
                    const uint32_t ones = take >= 32 ? 0xFFFFFFFFu : ((1u << take) - 1u);
                    er[ER_MASK + 3 * s + limb] |= ones << sh;
                    amount[s] = sh;
                }
                if (xr[XR_MASK] | xr[XR_MASK + 1] | xr[XR_MASK + 2]) {   // slot 7 holds the 1-bit fields of all limbs
                    for (uint32_t k = 0; k < 3; ++k) er[ER_MASK + 21 + k] = xr[XR_MASK + k];
                    amount7[0] = 0;
                    amount7[1] = (32u - ((cfg >> XC_ROT1_POS) & 31u)) & 31u;
                    amount7[2] = (32u - ((cfg >> XC_ROT2_POS) & 31u)) & 31u;
                }
            }
            for (uint32_t s = 0; s < 6; ++s) rot_a[r] |= amount[s] << (5 * s);
            rot_b[r] = amount[6] | (amount7[0] << 5) | (amount7[1] << 10) | (amount7[2] << 15);
        }
        for (size_t vi = 0; vi < nv; ++vi) {
            const uint32_t* er = &ft.enc[size_t(ext_of[vi]) * ER_WORDS];
            uint32_t need = 0;
            for (uint32_t q = 0; q < 6; ++q)
                if (er[4 * q] | er[4 * q + 1] | er[4 * q + 2] | er[4 * q + 3]) need |= 1u << q;
            ft.var[vi * VR_WORDS + VR_EXT] |= need << 16;
            ft.var[vi * VR_WORDS + VR_ROT_A] = rot_a[ext_of[vi]];
            ft.var[vi * VR_WORDS + VR_ROT_B] = rot_b[ext_of[vi]];
        }
    }

    // Buckets on and_base bits 11:0, then the split tree inside each bucket.  Variants that
    // can never match (constant ones above bit 95) still make their opcode bits "known".
    std::vector<std::vector<uint32_t>> buckets(4096);
    std::vector<uint32_t> bucket_size(4096, 0);
    for (size_t vi = 0; vi < nv; ++vi) {
        const size_t b = size_t(t.variants[vi].and_base & 0xFFF);
        ft.max_bucket = std::max(ft.max_bucket, ++bucket_size[b]);
        if (st[vi].matchable()) buckets[b].push_back(uint32_t(vi));
    }
    std::vector<uint32_t> dir(4096, 0);
    TreeBuilder tb{st, ext_of, ft};
    tb.class_budget = 2 * nv + 256;
    for (size_t b = 0; b < 4096; ++b) {
        if (!bucket_size[b]) continue;
        ++ft.n_buckets;
        dir[b] = buckets[b].empty() ? uint32_t(REF_LEAF) : tb.build(buckets[b], 0xFFF, 0);
    }
    tb.flatten_all(dir);
    ft.max_depth = tb.max_depth;
    // An empty leaf (opcode bits that only unmatchable variants have, an unused entry of a hash
    // node's child table) becomes a leaf of one class that never matches, so that every leaf the
    // kernels reach has a first class to test.
    {
        const uint32_t never = uint32_t(ft.classes.size() / CR_WORDS);
        if (never >= (1u << 20)) throw std::runtime_error("match tree too large");
        uint32_t rec[CR_WORDS] = {0};
        rec[CR_SBASE] = 0x10000u;   // (cc & 0) ^ base is never 0
        ft.classes.insert(ft.classes.end(), rec, rec + CR_WORDS);
        const uint32_t empty = REF_LEAF, filled = REF_LEAF | never | (1u << 20);
        for (uint32_t& r : dir) if (r == empty) r = filled;
        for (uint32_t& r : ft.children) if (r == empty) r = filled;
    }
    if (ft.broad.empty()) ft.broad.assign(BR_WORDS, 0);

    // One blob: hot sections first, each 16-byte aligned.
    auto place = [&](const std::vector<uint32_t>& src) {
        while (ft.blob.size() % 4) ft.blob.push_back(0);
        const uint32_t at = uint32_t(ft.blob.size());
        ft.blob.insert(ft.blob.end(), src.begin(), src.end());
        return at;
    };
    BlobLayout& L = ft.at;
    L.dir = place(dir);
    // Quad `q` of every record of a section whose records are `words` wide.
    auto quad_plane = [](const std::vector<uint32_t>& src, size_t words, size_t q) {
        std::vector<uint32_t> out;
        for (size_t r = 0; r * words < src.size(); ++r) out.insert(out.end(), src.begin() + r * words + 4 * q, src.begin() + r * words + 4 * q + 4);
        return out;
    };
    for (size_t q = 0; q < 2; ++q) L.nodes[q] = place(quad_plane(ft.nodes, NR_WORDS, q));
    L.children = place(ft.children);
    // Words [first, first + count) of every record of a section whose records are `words` wide.
    auto word_plane = [](const std::vector<uint32_t>& src, size_t words, size_t first, size_t count) {
        std::vector<uint32_t> out;
        for (size_t r = 0; r * words < src.size(); ++r) out.insert(out.end(), src.begin() + r * words + first, src.begin() + r * words + first + count);
        return out;
    };
    L.classes[0] = place(word_plane(ft.classes, CR_WORDS, CR_SMASK, 4));       // mask[3], base[0]
    L.classes[1] = place(word_plane(ft.classes, CR_WORDS, CR_SBASE + 1, 2));   // base[1], base[2]
    L.classes[2] = place(quad_plane(ft.classes, CR_WORDS, 2));
    L.class_info = place(word_plane(ft.classes, CR_WORDS, CR_INFO, 2));
    for (size_t q = 0; q < 2; ++q) L.broad[q] = place(quad_plane(ft.broad, BR_WORDS, q));
    while (ft.blob.size() % 4) ft.blob.push_back(0);
    L.sel_words = uint32_t(ft.blob.size());   // the roundtrip kernel stages up to here
    for (size_t q = 0; q < XR_WORDS / 4; ++q) L.ext[q] = place(quad_plane(ft.ext, XR_WORDS, q));
    while (ft.blob.size() % 4) ft.blob.push_back(0);
    L.hot_words = uint32_t(ft.blob.size());
    L.classes[3] = place(quad_plane(ft.classes, CR_WORDS, 3));   // read only when rank keys are compared: not staged
    L.enc_stride = uint32_t(ft.enc.size() / ER_WORDS * 4);
    for (size_t q = 0; q < ER_WORDS / 4; ++q) {
        const uint32_t at = place(quad_plane(ft.enc, ER_WORDS, q));
        if (q == 0) L.enc = at;
    }
    for (size_t q = 0; q < 2; ++q) L.var[q] = place(quad_plane(ft.var, VR_WORDS, q));
    while (ft.blob.size() % 4) ft.blob.push_back(0);
    L.enc_end = uint32_t(ft.blob.size());
    L.flagbest = place(ft.flagbest);
    ft.leafbest.resize(std::max<size_t>(ft.leafbest.size(), (ft.classes.size() / CR_WORDS) * FB_WORDS), 0);
    L.leafbest = place(ft.leafbest);
    L.gfields = place(ft.gfields);
    L.metaf = place(ft.metaf);
    L.gindex = place(ft.gindex);
    L.rt[0] = place(ft.rt);
    L.rt[1] = place(ft.rt_masks);
    while (ft.blob.size() % 4) ft.blob.push_back(0);
    L.total_words = uint32_t(ft.blob.size());
    L.n_variants = uint32_t(nv);
    return ft;
}

// ---- synthetic stream tables -------------------------------------------------------------

SynthTables build_synth_tables(const IsaTable& t, uint32_t mix, uint64_t seed) {
    std::vector<uint32_t> keys;   // keys that have at least one variant, bytewise order
    for (uint32_t k = 0; k < t.keys.size(); ++k)
        if (t.keys[k].n_variants) keys.push_back(k);
    const size_t n = keys.size();
    if (n == 0) throw std::runtime_error("table has no encodable key");
    SynthTables s;
    s.cdf.resize(n);
    std::vector<uint32_t> order(keys);
    const u128 kTotal = (u128)1 << 64;
    if (mix == MIX_UNIFORM) {
        for (size_t r = 0; r < n; ++r) s.cdf[r] = uint64_t((kTotal * (r + 1)) / n - 1);
    } else if (mix == MIX_ZIPF) {
        // Fisher-Yates over the key list, then Zipf(s = 1.1) mass by rank.
        for (size_t i = n - 1; i > 0; --i) {
            const size_t j = size_t(synth_draw(seed, ~0ull, i) % (i + 1));
            std::swap(order[i], order[j]);
        }
        std::vector<double> w(n);
        double total = 0;
        for (size_t r = 0; r < n; ++r) { w[r] = std::pow(double(r + 1), -1.1); total += w[r]; }
        double cum = 0;
        uint64_t prev = 0;
        for (size_t r = 0; r < n; ++r) {
            cum += w[r];
            const double frac = cum / total;
            uint64_t thr = frac >= 1.0 ? ~0ull : uint64_t(std::ldexp(frac, 64));
            if (thr > 0) --thr;
            if (thr < prev) thr = prev;
            s.cdf[r] = thr;
            prev = thr;
        }
    } else if (mix == MIX_FAMILY) {
        // 40% tensor-core MMA keys, 25% global/shared memory keys, 35% everything else.
        std::vector<uint32_t> grp[3];
        for (uint32_t k : keys) {
            const std::string b = base_op_of(t.keys[k].name);
            if (b == "QMMA" || b == "HMMA" || b == "IMMA") grp[0].push_back(k);
            else if (b == "LDG" || b == "LDS" || b == "STG" || b == "LDGSTS") grp[1].push_back(k);
            else grp[2].push_back(k);
        }
        const u128 mass[3] = {kTotal * 40 / 100, kTotal * 25 / 100, kTotal - kTotal * 40 / 100 - kTotal * 25 / 100};
        order.clear();
        u128 base = 0;
        size_t r = 0;
        for (int g = 0; g < 3; ++g) {
            for (size_t i = 0; i < grp[g].size(); ++i, ++r) {
                order.push_back(grp[g][i]);
                s.cdf[r] = uint64_t(base + (mass[g] * (i + 1)) / grp[g].size() - 1);
            }
            if (!grp[g].empty()) base += mass[g];
        }
    } else {
        throw std::runtime_error("unknown synthetic mix");
    }
    s.cdf[n - 1] = ~0ull;
    for (uint32_t k : order) {
        s.rank_first.push_back(t.keys[k].first_variant);
        s.rank_count.push_back(t.keys[k].n_variants);
    }
    return s;
}

}  // namespace cubit
