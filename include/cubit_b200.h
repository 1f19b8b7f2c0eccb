/*
 * cubit_b200 — C ABI of the B200 batch SM120 SASS codec.
 *
 * The reference (kacper-daftcode/cubit, a Rust crate) exposes this path only through its
 * Rust library API and a PyO3 module; it has no C ABI of its own.  Each entry point below
 * names the reference interface it stands in for.  All functions return 0 on success or a
 * negative cubit_status; none of them throws or aborts.  The caller owns every buffer.
 * A context is immutable after creation and may be used from several host threads at once.
 *
 * Words are 16 bytes, little-endian: bytes 0..7 = lo64, bytes 8..15 = hi64
 * (reference src/python.rs:127-129).
 *
 * A decoded record is structure-of-arrays:
 *   form  u16[n]      variant id (index of (key, mod_group) in bytewise order), 0xFFFF = rejected
 *   slots u32[8][n]   slot-major: slot s of record i is slots[s * n + i]
 *   ctrl  u32[n]      [16:0] scheduling word (wait|rbar|wbar|yield|stall), [19:17] reuse bits,
 *                     [23:20] guard nibble, [27:24] synthesized abs/neg presence (bits 63,62,72,73),
 *                     [28] tie, [31:30] status (0 ok, 1 unknown opcode bits, 2 no variant matches)
 * Where each table field of a variant lives inside the 8 slots is static per variant and
 * reported by cubit_variant_lookup (cubit_field_info.dst_pos / stored_bits).  The decoder reads
 * fields from the word with bits 127:96 cleared, so field bits at or above bit 96 are always
 * zero and are not stored.
 */
#ifndef CUBIT_B200_H
#define CUBIT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cubit_ctx cubit_ctx;
typedef struct cubit_elf cubit_elf;

typedef enum {
    CUBIT_OK = 0,
    CUBIT_ERR_INVALID = -1,    /* bad argument */
    CUBIT_ERR_TABLE = -2,      /* ISA table missing, malformed or too large */
    CUBIT_ERR_CUDA = -3,       /* a CUDA call failed; see cubit_last_error */
    CUBIT_ERR_NO_DEVICE = -4,  /* compute entry point called on a context without a GPU */
    CUBIT_ERR_ELF = -5,        /* not a little-endian ELF64, or truncated */
    CUBIT_ERR_NOT_FOUND = -6,  /* kernel / variant name not found */
    CUBIT_ERR_NOMEM = -7,
    CUBIT_ERR_TEXT = -8        /* SASS text did not parse, or no table entry fits its operands */
} cubit_status;

enum { CUBIT_MEM_HOST = 0, CUBIT_MEM_DEVICE = 1 };
enum { CUBIT_MIX_UNIFORM = 0, CUBIT_MIX_ZIPF = 1, CUBIT_MIX_FAMILY = 2 };
enum { CUBIT_FORM_NONE = 0xFFFF };
enum { CUBIT_RT_EXACT = 0, CUBIT_RT_MISMATCH = 1, CUBIT_RT_REJECTED = 2 };

typedef struct {
    uint64_t n_decoded;   /* decode / roundtrip: words that selected a variant */
    uint64_t n_rejected;  /* words that match no variant */
    uint64_t n_tie;       /* decoded words whose winner was separated only by canonical order */
    uint64_t n_exact;     /* roundtrip: re-encoded word equals the input outside bits 121:105 */
    uint64_t n_mismatch;  /* roundtrip: it does not */
} cubit_counts;

typedef struct {
    uint32_t shift, bits;
    int32_t token_idx;
    uint32_t dst_pos;        /* bit position of the value in the 256-bit slot area (slot = pos/32);
                                0xFFFFFFFF when the field lies at or above bit 96 and is never stored */
    uint32_t stored_bits;    /* bits of the field below bit 96 of the word: the width held at dst_pos */
    const char* name;        /* "Rd", "Ra", "Rb", "Rc", "guard" or "[hi:lo]" */
    const char* extraction;  /* spelling reported by the reference decoder */
} cubit_field_info;

typedef struct {
    const char* key;
    const char* mod_group;
    const char* opcode;
    uint32_t key_id;
    uint32_t layout_kind;    /* 0 = one slot per multi-bit field, 1-bit fields share slot 7;
                                1 = field bits stay at their word position (slot k = bits 32k+31:32k) */
    uint32_t synth_mask;     /* which of bits 63, 62, 72, 73 can carry a synthesized neg/abs */
    int32_t ra_tok, rb_tok;  /* token index reported for synthesized Ra / Rb modifiers */
    uint32_t n_fields;
    const cubit_field_info* fields;
} cubit_variant_info;

/* ---- context ------------------------------------------------------------------------ */

/* Replaces IsaTable::load_default + DecodeIndex::build (reference src/table.rs:239-249,
 * src/decoder.rs:80-160; the process-global pair of src/python.rs:28-42).  Table source:
 * $CUBIT_TABLE if set (strict), else `table_path`, else the copy bundled with the library.
 * The table is compiled to flat arrays and uploaded to each listed CUDA device.
 * n_devices == 0 gives a host-only context: metadata and ELF helpers work, compute entry
 * points return CUBIT_ERR_NO_DEVICE.  On failure *out is NULL and cubit_last_error(NULL)
 * describes why. */
int cubit_ctx_create(const char* table_path, const int* devices, int n_devices, cubit_ctx** out);
void cubit_ctx_destroy(cubit_ctx* ctx);

/* Message of the last failure on this thread for `ctx` (NULL: for cubit_ctx_create / ELF helpers).
 * Mirrors the reference's anyhow error strings (src/decoder.rs:173, :287). */
const char* cubit_last_error(const cubit_ctx* ctx);

/* Replaces table_info() (reference src/python.rs:171-177): (2001, 2872) for the bundled table. */
int cubit_table_info(const cubit_ctx* ctx, uint32_t* n_keys, uint32_t* n_groups);

/* Static description of one variant: what a host needs to rebuild the reference's DecodedInst
 * (src/decoder.rs:32-47) from a record.  Pointers stay valid until cubit_ctx_destroy. */
int cubit_variant_lookup(const cubit_ctx* ctx, uint32_t variant, cubit_variant_info* out);
/* Replaces IsaTable::get (reference src/table.rs:406-408). */
int cubit_variant_find(const cubit_ctx* ctx, const char* key, const char* mod_group, uint32_t* variant);
int cubit_key_name(const cubit_ctx* ctx, uint32_t key_id, const char** name, uint32_t* first_variant,
                   uint32_t* n_variants);

/* Pinned host memory for the CUBIT_MEM_HOST paths (plain malloc'd memory also works, slower). */
int cubit_host_alloc(cubit_ctx* ctx, uint64_t bytes, void** out);
int cubit_host_free(cubit_ctx* ctx, void* p);

/* ---- batch codec ---------------------------------------------------------------------- */

/* Replaces a loop of DecodeIndex::decode (reference src/decoder.rs:163-382) over n words.
 * mem_kind HOST: buffers are host memory; the words are split into contiguous ranges over
 * the context's devices, copied in, decoded and copied back.  DEVICE: buffers live on one of
 * the context's devices and the kernel is queued on `stream` (a cudaStream_t, NULL = default);
 * the call returns without waiting unless `counts` is given.  `counts` may be NULL. */
int cubit_decode_batch(cubit_ctx* ctx, const void* words, uint64_t n, uint16_t* form, uint32_t* slots,
                       uint32_t* ctrl, cubit_counts* counts, int mem_kind, void* stream);

/* Record -> word: the table-driven core of encode_instruction (reference src/encoder.rs:293-300,
 * :341-384, :530-532, :560-608, :1155-1179) applied to records instead of parsed text.
 * form >= number of variants gives a zero word. */
int cubit_encode_batch(cubit_ctx* ctx, const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl,
                       uint64_t n, void* words, int mem_kind, void* stream);

/* Fused decode -> encode -> compare outside the scheduling field, the per-word faithfulness
 * check of the reference (src/main.rs:270, :578-581, :717-737) at record level.
 * status[i] is CUBIT_RT_EXACT / MISMATCH / REJECTED. */
int cubit_roundtrip_batch(cubit_ctx* ctx, const void* words, uint64_t n, uint8_t* status,
                          cubit_counts* counts, int mem_kind, void* stream);

/* Seeded synthetic instruction stream, words [first, first + n) of the stream (mix, seed,
 * noise_ppm); any range can be produced on its own, so shards of one stream agree bit for bit.
 * words / form / slots / ctrl may each be NULL.  Records are the generator's own (the input of
 * an encode benchmark); noise words have form 0xFFFF.  No counterpart in the reference, whose
 * corpus is private. */
int cubit_synth_batch(cubit_ctx* ctx, uint32_t mix, uint64_t seed, uint32_t noise_ppm, uint64_t first,
                      uint64_t n, void* words, uint16_t* form, uint32_t* slots, uint32_t* ctrl,
                      int mem_kind, void* stream);

/* Largest batch cubit_decode_batch_static accepts. */
#define CUBIT_STATIC_MAX_WORDS 65536

/* Host-buffer decode that allocates nothing (no counterpart in the reference, which has no
 * device memory to manage).  It is for callers that must not allocate device memory once they
 * are running: a process in which another component has already reserved the GPU's memory, so
 * that cudaMalloc would fail, or a latency-critical thread that cannot afford the implicit
 * device synchronisation of cudaMalloc / cudaFree.  cubit_decode_batch grows a staging buffer
 * with cudaMalloc when it is handed host memory; this entry point stages through a fixed
 * array built into the library instead (about 3.4 MiB per GPU, held until the process exits),
 * and calls no cudaMalloc, cudaFree or other allocating routine.
 *   - words / form / slots / ctrl are host buffers as for cubit_decode_batch(CUBIT_MEM_HOST),
 *     slots being u32[8][n]; results are identical to cubit_decode_batch's.
 *   - n above CUBIT_STATIC_MAX_WORDS is refused with CUBIT_ERR_INVALID.
 *   - device_slot picks one of the context's devices by position in the list given to
 *     cubit_ctx_create.  The first call on a device looks up the array's address there
 *     (a one-time set-up); make that first call before starting any stream capture.
 *   - All calls on one GPU share the array, whichever context they come from: it exists once
 *     per GPU and process.  It keeps the previous call's contents; the entry point clears the
 *     counters it accumulates into and overwrites the rest.  Calls that overlap in time on the
 *     same GPU would race on it, so the library serialises them with one lock per GPU that all
 *     contexts of the process share (and, within a context, with the CUBIT_MEM_HOST paths,
 *     which use the same staging stream).  Another process, or another copy of the library
 *     loaded into this one, has an array of its own.
 * The call returns when the results are in the host buffers. */
int cubit_decode_batch_static(cubit_ctx* ctx, int device_slot, const void* words, uint64_t n, uint16_t* form,
                              uint32_t* slots, uint32_t* ctrl, cubit_counts* counts);

/* ---- cubin (ELF) ------------------------------------------------------------------------ */

/* Replaces CubinFile::from_bytes (reference src/elf.rs:29-58): lists PROGBITS sections named
 * ".text" or ".text.*" with size > 0, in section-header order.  `bytes` must outlive the handle. */
int cubit_elf_parse(const void* bytes, uint64_t len, cubit_elf** out);
void cubit_elf_free(cubit_elf* elf);
uint32_t cubit_elf_num_text(const cubit_elf* elf);
int cubit_elf_text(const cubit_elf* elf, uint32_t index, const char** name, uint64_t* offset, uint64_t* size);
/* First text section whose name contains `kernel_name` (reference src/python.rs:113-114). */
int cubit_elf_find(const cubit_elf* elf, const char* kernel_name, uint32_t* index);

/* Replaces the per-word loop of decode_kernel (reference src/python.rs:124-167) for many
 * kernels at once: every 16-byte word of the chosen text sections (indices == NULL: all) is
 * decoded in one launch per device.  word_start[k] (n_sections + 1 entries, output) is the
 * record index of the first word of section k; a trailing partial word is ignored.
 * Output buffers are host memory with room for `capacity` records; `raw_words` (optional)
 * receives the 16-byte words in record order.  Call with form == NULL to get only word_start. */
int cubit_decode_elf(cubit_ctx* ctx, const cubit_elf* elf, const uint32_t* indices, uint32_t n_sections,
                     uint64_t* word_start, uint64_t capacity, uint16_t* form, uint32_t* slots,
                     uint32_t* ctrl, void* raw_words, cubit_counts* counts);

typedef struct {
    uint32_t regcount;      /* (max_reg + 32) & ~31, at least 32: registers are allocated in blocks of 32 */
    uint32_t num_barriers;  /* distinct BSSY barrier indices */
    uint32_t max_reg;       /* largest register number below 255 named by the code */
    uint32_t barrier_mask;  /* bit b set: barrier b is used */
    uint64_t first_exit;    /* index of this kernel's first entry in exit_offsets */
    uint64_t n_exits;       /* number of EXIT instructions */
} cubit_kernel_meta;

/* Replaces infer_kernel_meta (reference src/main.rs:787-867) for many kernels at once: one
 * launch decodes every word of the chosen text sections (indices == NULL: all) and reduces,
 * per kernel, the largest register number, the BSSY barrier set and the EXIT positions; words
 * that match no variant use the reference's raw-bits fallback.  exit_offsets (optional)
 * receives the byte offsets of EXIT instructions inside their section, kernel by kernel in
 * ascending order; *n_exits is their total (call with exit_offsets == NULL to size it). */
int cubit_infer_kernel_meta(cubit_ctx* ctx, const cubit_elf* elf, const uint32_t* indices, uint32_t n_sections,
                            cubit_kernel_meta* meta, uint32_t* exit_offsets, uint64_t exit_capacity,
                            uint64_t* n_exits);

/* Synthetic multi-kernel cubin with the section layout of the reference's Mercury-free
 * builder (src/elf_builder.rs:535-847): 9 + 4N sections, one ".text.<name>" per kernel,
 * 128-byte aligned and padded with NOPs plus one trailing self-branch.  Note and info
 * sections carry placeholder contents; the result is an input for cubit_elf_parse, not a
 * loadable module.  Call with out == NULL to get the required size in *out_len. */
int cubit_elf_build(const char* const* names, const void* const* code, const uint64_t* code_bytes,
                    uint32_t n_kernels, void* out, uint64_t capacity, uint64_t* out_len);

/* ---- SASS text (host) -------------------------------------------------------------------- */

/* Text is handled on the host; only the table-driven part of an encode runs on the GPU.  An
 * instruction's text is lowered to a record (form, slots, ctrl, as cubit_encode_batch takes)
 * plus a 128-bit patch: the bits the reference derives from the text itself and not from
 * table fields (branch targets, register placement fixups, raw-address LDG/STG, the control
 * word).  The encoded word is (cubit_encode_batch word & ~clear) | set.
 *
 * `mode` CUBIT_TEXT_ONE: `text` is one bare instruction, parsed as parse_sass does (reference
 *   src/parser.rs:358-478); failures set "parse error: ..." / "encode error: ..." as the
 *   reference's Python encode() raises them (src/python.rs:48-55).
 * `mode` CUBIT_TEXT_PROGRAM: statements separated by ';' or newlines, optional
 *   "[B------:R-:W-:-:S01]" control prefixes, "name:" labels resolved to branch targets,
 *   // and # comments, unparsable lines skipped (parse_multi_sass + resolve_labels, reference
 *   src/parser.rs:485-588); instruction k sits at base_addr + 16 k.  A "__raw__0x<hex>"
 *   statement is emitted unchanged (reference src/main.rs:1918-1927).  The reference's
 *   assemble() additionally runs its scheduling pass over the control codes
 *   (src/lib.rs:52-54); that pass is not part of this library, control codes are taken as
 *   written (default B------:R-:W-:-:S01).
 * Deviation: the reference numbers ".?<n>" opaque modifiers with a counter that is not reset
 * when the same text is encoded twice in a row (src/encoder.rs:1036-1045); here every
 * instruction starts at its first value. */
enum { CUBIT_TEXT_ONE = 0, CUBIT_TEXT_PROGRAM = 1 };

/* Lowers text to records and patches.  Buffers hold `capacity` instructions; slots is
 * slot-major with stride `capacity` (slot s of instruction i at slots[s * capacity + i]);
 * clear / set are `capacity` x 16 bytes, little-endian.  *n_out is the instruction count; when
 * it exceeds capacity (or a buffer is NULL) nothing is written and CUBIT_OK is returned, so a
 * first call with capacity 0 sizes the buffers.  Works on a context without a GPU. */
int cubit_text_lower(cubit_ctx* ctx, const char* text, uint32_t base_addr, int mode, uint64_t capacity,
                     uint16_t* form, uint32_t* slots, uint32_t* ctrl, void* clear, void* set, uint64_t* n_out);

/* Replaces encode(sass, addr) (reference src/python.rs:48-60, CUBIT_TEXT_ONE) and the encode
 * loop of cubit::assemble (src/lib.rs:49-63, CUBIT_TEXT_PROGRAM): lowers the text, encodes the
 * records with the batch kernel and applies the patches.  `words` is host memory for
 * `capacity` x 16 bytes; sizing works as for cubit_text_lower. */
int cubit_text_encode(cubit_ctx* ctx, const char* text, uint32_t base_addr, int mode, uint64_t capacity,
                      void* words, uint64_t* n_out);

/* The parsed form of one instruction as JSON, for tools and tests: {"key", "opcode",
 * "opcode_full", "mod_group", "guard": null | {"pred", "negated", "uniform"}, "modifiers",
 * "ctrl": "B------:R-:W-:-:S01", "hand_sched", "operands": [{"type": "R", "kind": "Reg", ...}]}.
 * `line` may carry a control prefix (parse_cuasm_line, reference src/parser.rs:591-604).
 * *needed is the length including the terminating NUL; nothing is written when it exceeds
 * capacity. */
int cubit_text_parse(cubit_ctx* ctx, const char* line, uint32_t addr, char* json, uint64_t capacity,
                     uint64_t* needed);

/* Replaces printer::to_sass (reference src/printer.rs:12) and to_sass(lo, hi, addr) (src/python.rs:186-197)
 * for a batch: prints word i, located at base_addr + 16 i (branch targets are absolute), as one
 * line of SASS text without the trailing " ;", each line ended by '\n'.  form / slots / ctrl
 * are the records of the words as cubit_decode_batch wrote them (slots slot-major, stride n);
 * pass all three NULL to have the words decoded here (needs a GPU).  A word that matches no
 * variant prints as the disassembler's placeholder comment with the word in hex (reference
 * src/main.rs:497).  All buffers are host memory.  *needed is the text length including the
 * terminating NUL; nothing is written when it exceeds capacity. */
int cubit_text_print(cubit_ctx* ctx, const void* words, uint64_t n, uint32_t base_addr, const uint16_t* form,
                     const uint32_t* slots, const uint32_t* ctrl, char* out, uint64_t capacity, uint64_t* needed);

/* Replaces cmd_disassemble (reference src/main.rs:401-627): a listing of every text section of
 * the cubin (or only the kernel whose name, without the ".text." prefix, equals only_kernel).
 * All words are decoded in one launch per device and printed on the host.
 *   frozen == 0: "// <kernel>", an optional "    .shared smem[N]", then one line per word,
 *     "  / *addr* /  <text> / * @sched 0x<5 hex> * / ;" (written without the spaces inside the
 *     comment marks), or the placeholder comment for a word that matches no variant.
 *   frozen != 0: a re-assemblable ".entry" block: ".reg", ".param" and ".shared" lines from the
 *     kernel's .nv.info / .nv.shared sections, "L_<addr>:" labels on branch targets, every
 *     instruction prefixed with its control code "[B------:R-:W-:-:S01]".  Each printed line is
 *     checked the way the reference does: its text is parsed and encoded again (one batch on
 *     the GPU) and must equal the original word outside the scheduling field; lines that fail,
 *     and words that match no variant, are emitted as "__raw__0x<32 hex> ;".  *n_raw (optional)
 *     counts those lines.
 * *needed is the text length including the terminating NUL; nothing is written when it
 * exceeds capacity. */
int cubit_disassemble(cubit_ctx* ctx, const cubit_elf* elf, const char* only_kernel, int frozen, char* out,
                      uint64_t capacity, uint64_t* needed, uint64_t* n_raw);

/* Replaces the encode loop of the reference's listing assembler (parse_sass_file_full,
 * src/main.rs:225-268, and cmd_asm_build_elf, src/main.rs:997-1075): reads a plain listing as
 * cubit_disassemble(frozen = 0) writes it -- "// <kernel>" headers, one
 * "  / *addr* /  <text> / * @sched 0x..... * / ;" line per instruction (comment marks without the
 * spaces), placeholder comments for undecodable words -- and produces the code bytes of `kernel`:
 * every line is parsed and encoded at its own address (one batch on the GPU), the "@sched" value
 * replaces the scheduling field (a line without one gets the reference's default dependency
 * rule: write barrier 1 when the first operand is a register, the instruction has no guard and
 * is not a store, branch or barrier, src/main.rs:766-783), a placeholder line contributes its raw
 * word.  Lines that do not parse or encode leave zero bytes and are counted in *n_failed.
 * The result is what cubit_elf_patch_text splices into a template cubin.  *needed is the code
 * length (highest address + 16); nothing is written when it exceeds capacity. */
int cubit_listing_assemble(cubit_ctx* ctx, const char* listing, const char* kernel, void* code, uint64_t capacity,
                           uint64_t* needed, uint64_t* n_failed);

/* ---- cubin rewriting ----------------------------------------------------------------------- */

typedef struct {
    uint64_t n_words;      /* instruction words in the chosen text sections */
    uint64_t n_reencoded;  /* words whose printed text parsed and encoded: their low 64 bits were rewritten */
    uint64_t n_kept;       /* words left as they were: no variant matches, or the text does not encode */
    uint64_t n_changed;    /* re-encoded words whose low 64 bits differ from the original */
    uint64_t n_unfaithful; /* re-encoded words that differ from the original outside the scheduling field */
} cubit_patch_stats;

/* Replaces cmd_patch (reference src/main.rs:691-764): every word of every text section goes
 * decode -> print -> parse -> encode; where that succeeds the word's low 64 bits are replaced by
 * the re-encoded ones and its high 64 bits are kept (src/main.rs:740-746), otherwise the word is
 * kept.  Here: one decode launch per device over all sections, printing and lowering on the
 * host, one encode launch.  `out` receives the whole file (same length as the input);
 * *needed is that length, nothing is written when it exceeds capacity. */
int cubit_patch_elf(cubit_ctx* ctx, const cubit_elf* elf, void* out, uint64_t capacity, uint64_t* needed,
                    cubit_patch_stats* stats);

/* Replaces CubinFile::patch_text (reference src/elf.rs:71-219): the file with text section
 * `index` (as numbered by cubit_elf_text) replaced by `code`.  A different length splices the
 * file and moves every offset behind the section (section and program headers, e_shoff / e_phoff,
 * sizes of the section's symbols, a DWARF64 .debug_frame range equal to the old size).
 * *needed is the new file length; nothing is written when it exceeds capacity. */
int cubit_elf_patch_text(const cubit_elf* elf, uint32_t index, const void* code, uint64_t code_len, void* out,
                         uint64_t capacity, uint64_t* needed);

#ifdef __cplusplus
}
#endif
#endif /* CUBIT_B200_H */
