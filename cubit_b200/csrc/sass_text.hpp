// Host text layer: SASS text -> typed instruction -> (record, patch) for the batch encoder.
//
// Mirrors the behaviour of the reference's parser (src/parser.rs) and of the text-semantic
// half of its encoder (src/encoder.rs:42-258 lookup chain and operand checks, :615-1060
// operand -> field value conversions, :395-443 register placement fixups, :1069-1146 branch
// targets, :468-516 raw-address LDG/STG, :1181-1215 PLOP3 / FADD fixups, :560-608 control
// word).  Text never goes to the GPU: an instruction is lowered to
//   * a record (variant id, one value per table field, guard nibble, reuse bits, scheduling)
//     that the batch encode kernel turns into and_base | fields | guard | reuse | control, and
//   * a patch (clear mask, set value) holding every bit the reference derives from the text
//     rather than from table fields; the final word is (kernel word & ~clear) | set.
#pragma once
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "isa_table.hpp"

namespace cubit {

// Message texts follow the reference's ("unrecognized SASS: ...", "no operand-compatible
// table entry; attempted keys: [...]", "invalid control code string: ...").
struct TextError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

enum class OperandKind : uint8_t {
    Reg, UReg, Pred, UPred, Imm32, Imm64, FloatImm, Addr, ConstMem, Desc, BranchTarget, Barrier, SysReg, Label,
};

// One typed operand (reference src/ir.rs:38-84).  Only the members of its kind are meaningful.
struct TextOperand {
    OperandKind kind = OperandKind::Label;
    uint8_t num = 0;                       // register / predicate / barrier number (RZ = 255, URZ = 63, PT = 7)
    bool neg = false, abs = false, inv = false, reuse = false, is_zero = false;
    int64_t imm = 0;                       // Imm32
    uint64_t bits = 0;                     // Imm64 value, FloatImm as f64 bits
    bool has_base = false; uint8_t base = 0;      // Addr / ConstMem / Desc base register
    bool has_suffix = false; std::string suffix;  // ".64"-style suffix of the base register, without the dot
    bool has_ur = false; uint8_t ur = 0;          // Addr / ConstMem uniform register
    uint16_t bank = 0;                     // ConstMem
    uint8_t ur_idx = 0;                    // Desc
    int64_t offset = 0;
    uint32_t target = 0;                   // BranchTarget (absolute byte offset)
    std::string text;                      // SysReg name, Label text
};

struct TextControl {                       // reference src/ir.rs:17-36 and its defaults
    uint8_t stall = 1;
    bool yield_flag = false;
    uint8_t write_bar = 7, read_bar = 7, wait_mask = 0;
};

struct TextInstruction {                   // reference src/ir.rs:87-113
    uint32_t addr = 0;
    std::string opcode, opcode_full, key;
    bool has_guard = false;
    uint8_t guard_pred = 7; bool guard_neg = false, guard_uniform = false;
    std::vector<TextOperand> operands;
    std::vector<std::string> modifiers;
    TextControl ctrl;
    bool hand_sched = false;
    std::string raw_text;
};

// "B------:R-:W-:-:S01" <-> TextControl (reference src/scheduling.rs:31-100).
TextControl parse_control_code(const std::string& s);
std::string format_control_code(const TextControl& c);
uint32_t pack_control_code(const TextControl& c);   // the 17-bit scheduling value, not shifted
TextControl unpack_control_code(uint32_t sched17);

const char* operand_type_label(const TextOperand& op);

// One instruction, bare (parse_sass) or with a "[B..:R.:W.:.:S..]" prefix (parse_cuasm_line).
TextInstruction parse_sass(const std::string& text, uint32_t addr);
TextInstruction parse_cuasm_line(const std::string& line, uint32_t addr);
// Several statements separated by ';' or newlines, with "name:" labels and // or # comments;
// lines that do not parse are skipped, labels of branch operands resolve to addresses
// (reference src/parser.rs:485-588, both passes).
// `runner(n, body)` must call body(begin, end) over ranges covering [0, n), possibly from several
// threads: statements are parsed independently of one another; null runs them in order here.
typedef std::function<void(size_t, const std::function<void(size_t, size_t)>&)> RangeRunner;
std::vector<TextInstruction> parse_program(const std::string& text, uint32_t base_addr, const RangeRunner& runner = nullptr);

// Sorted, comma-joined dot-modifiers of the mnemonic (reference src/table.rs:477-502).
std::string extract_mod_group(const std::string& sass);

struct LoweredInstruction {
    bool raw = false;                // "__raw__0x..." statement: `set` is the whole word, nothing to encode
    uint32_t variant = 0;
    std::vector<uint64_t> values;    // one per table field of the variant, already masked
    uint32_t ctrl = 0;               // record control word: [16:0] scheduling, [19:17] reuse, [23:20] guard
    u128 clear = 0, set = 0;
};

// A decoded instruction as the printer reads it (reference src/decoder.rs:15-59): table fields
// with their decoded values in table order, then the synthesized neg / abs fields.
struct PrintField {
    uint32_t shift = 0, bits = 0;
    uint64_t value = 0;
    int32_t token_idx = 0;
    std::string ext;      // extraction name as the decoder reports it (reference src/decoder.rs:679-705)
};
// What the printer derives from a variant's names alone; callers that print many words build
// it once per variant.
struct VariantPrintCache {
    std::vector<std::string> op_types;   // operand-type segments of the key (reference src/printer.rs:345-370)
    std::string mnemonic;                // opcode + ordered modifiers (reference src/printer.rs:430-445)
};
VariantPrintCache make_print_cache(const std::string& key, const std::string& opcode, const std::string& mod_group);

struct DecodedView {
    std::string key, mod_group, opcode;
    std::vector<PrintField> fields;
    u128 raw = 0;
    uint32_t addr = 0;
    const VariantPrintCache* cache = nullptr;   // optional; computed on the fly when null
};
// SASS text without the trailing " ;" (reference src/printer.rs:12-212).
std::string to_sass(const DecodedView& insn);

class TextEncoder {
public:
    explicit TextEncoder(const IsaTable& table);
    // Throws TextError with the reference's message when no table entry fits the operands.
    LoweredInstruction lower(const TextInstruction& insn) const;
    // Variant id of (key, mod_group), -1 when the table has no such pair.
    int find(const std::string& key, const std::string& mod_group) const;

private:
    const IsaTable& table_;
    std::unordered_map<std::string, uint32_t> key_index_;
    const IsaVariant* get(const std::string& key, const std::string& mod_group, uint32_t* id) const;
};

}  // namespace cubit
