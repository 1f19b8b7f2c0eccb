// Cubin (ELF64, little-endian) text-section reader and a synthetic multi-kernel builder.
//
// Reader: what the reference's CubinFile::from_bytes keeps (src/elf.rs:29-58) — name, file
// offset and size of every PROGBITS section called ".text" or ".text.*" with size > 0.
// Builder: the section layout of the reference's Mercury-free writer
// (src/elf_builder.rs:535-847), enough for the reader and for benchmarks; note/info
// sections are placeholders.
#include "elf_text.hpp"

#include <cstring>
#include <stdexcept>

namespace cubit {

static uint16_t rd16(const uint8_t* p) { return uint16_t(p[0] | (p[1] << 8)); }
static uint32_t rd32(const uint8_t* p) { return uint32_t(p[0]) | (uint32_t(p[1]) << 8) | (uint32_t(p[2]) << 16) | (uint32_t(p[3]) << 24); }
static uint64_t rd64(const uint8_t* p) { return uint64_t(rd32(p)) | (uint64_t(rd32(p + 4)) << 32); }
static void wr16(uint8_t* p, uint16_t v) { p[0] = uint8_t(v); p[1] = uint8_t(v >> 8); }
static void wr32(uint8_t* p, uint32_t v) { for (int i = 0; i < 4; ++i) p[i] = uint8_t(v >> (8 * i)); }
static void wr64(uint8_t* p, uint64_t v) { for (int i = 0; i < 8; ++i) p[i] = uint8_t(v >> (8 * i)); }

static const uint32_t SHT_PROGBITS = 1, SHT_SYMTAB = 2, SHT_STRTAB = 3, SHT_NOTE = 7, SHT_NOBITS = 8;

std::vector<ElfSection> elf_sections(const uint8_t* b, uint64_t len) {
    if (len < 64 || memcmp(b, "\x7f" "ELF", 4) != 0) throw std::runtime_error("failed to parse ELF: bad magic");
    if (b[4] != 2) throw std::runtime_error("failed to parse ELF: not a 64-bit ELF");
    if (b[5] != 1) throw std::runtime_error("failed to parse ELF: not little-endian");
    const uint64_t shoff = rd64(b + 0x28);
    const uint16_t shentsize = rd16(b + 0x3A);
    uint64_t shnum = rd16(b + 0x3C);
    uint32_t shstrndx = rd16(b + 0x3E);
    std::vector<ElfSection> out;
    if (shoff == 0) return out;
    if (shentsize != 64) throw std::runtime_error("failed to parse ELF: unexpected section header size");
    if (shoff > len || len - shoff < 64) throw std::runtime_error("failed to parse ELF: section table past end of file");
    // Extended numbering: the real counts live in section header 0.
    if (shnum == 0) shnum = rd64(b + shoff + 0x20);
    if (shstrndx == 0xFFFF) shstrndx = rd32(b + shoff + 0x28);
    if (shnum > (len - shoff) / 64) throw std::runtime_error("failed to parse ELF: section table past end of file");
    if (shstrndx >= shnum) throw std::runtime_error("failed to parse ELF: bad section-name table index");
    const uint8_t* strsec = b + shoff + 64ull * shstrndx;
    if (rd32(strsec + 4) != SHT_STRTAB) throw std::runtime_error("failed to parse ELF: section-name table is not a string table");
    const uint64_t str_off = rd64(strsec + 0x18), str_size = rd64(strsec + 0x20);
    if (str_off > len || str_size > len - str_off) throw std::runtime_error("failed to parse ELF: section-name table past end of file");
    for (uint64_t i = 0; i < shnum; ++i) {
        const uint8_t* sh = b + shoff + 64 * i;
        const uint32_t name_off = rd32(sh);
        if (name_off >= str_size) continue;   // unreadable name: the section is skipped
        const char* name = (const char*)b + str_off + name_off;
        const void* nul = memchr(name, 0, size_t(str_size - name_off));
        if (!nul) continue;
        out.push_back(ElfSection{std::string(name, (const char*)nul - name), rd32(sh + 4), rd64(sh + 0x18), rd64(sh + 0x20)});
    }
    return out;
}

std::vector<TextSection> elf_text_sections(const uint8_t* b, uint64_t len) {
    std::vector<TextSection> out;
    for (const ElfSection& s : elf_sections(b, len)) {
        const bool is_text = s.name == ".text" || s.name.compare(0, 6, ".text.") == 0;
        if (is_text && s.type == SHT_PROGBITS && s.size > 0) out.push_back(TextSection{s.name, s.offset, s.size});
    }
    return out;
}

// ---- text replacement ----------------------------------------------------------------------

std::vector<uint8_t> elf_patch_text(const uint8_t* bytes, uint64_t len, uint32_t index, const uint8_t* code,
                                    uint64_t code_len) {
    const std::vector<TextSection> text = elf_text_sections(bytes, len);
    if (index >= text.size()) throw std::runtime_error("text section index out of range");
    const uint64_t start = text[index].offset, old_size = text[index].size;
    if (start > len || old_size > len - start)
        throw std::runtime_error("text section " + text[index].name + " extends past end of file");
    std::vector<uint8_t> out;
    out.reserve(len - old_size + code_len);
    out.insert(out.end(), bytes, bytes + start);
    out.insert(out.end(), code, code + code_len);
    out.insert(out.end(), bytes + start + old_size, bytes + len);
    if (code_len == old_size) return out;

    const int64_t delta = (int64_t)code_len - (int64_t)old_size;
    uint8_t* b = out.data();
    const uint64_t n = out.size();
    auto moved = [&](uint64_t v) { return (uint64_t)((int64_t)v + delta); };
    // [at, at + size) lies inside the image; written so that no sum can wrap.
    auto inside = [&](uint64_t at, uint64_t size) { return at <= n && size <= n - at; };
    if (n < 0x40) return out;
    if (rd64(b + 0x28) > start) wr64(b + 0x28, moved(rd64(b + 0x28)));
    if (rd64(b + 0x20) > start) wr64(b + 0x20, moved(rd64(b + 0x20)));
    const uint64_t shoff = rd64(b + 0x28), shnum = rd16(b + 0x3C), phoff = rd64(b + 0x20), phnum = rd16(b + 0x38);
    // A header table that starts outside the image cannot be fixed up.
    if ((phnum && phoff > n) || (shnum && shoff > n))
        throw std::runtime_error("failed to parse ELF: header table offset past end of file");
    for (uint64_t p = 0; p < phnum; ++p) {
        if (!inside(phoff, 56) || p > (n - phoff - 56) / 56) break;
        const uint64_t ph = phoff + p * 56;
        const uint64_t p_offset = rd64(b + ph + 8), p_filesz = rd64(b + ph + 0x20);
        if (p_offset <= start && start - p_offset < p_filesz) {
            wr64(b + ph + 0x20, moved(p_filesz));
            wr64(b + ph + 0x28, moved(rd64(b + ph + 0x28)));
        } else if (p_offset > start) {
            wr64(b + ph + 8, moved(p_offset));
        }
    }
    int64_t text_shndx = -1;
    for (uint64_t s = 0; s < shnum; ++s) {
        if (!inside(shoff, 64) || s > (n - shoff - 64) / 64) break;
        const uint64_t sh = shoff + s * 64;
        const uint64_t sh_offset = rd64(b + sh + 0x18), sh_size = rd64(b + sh + 0x20);
        if (sh_offset == start && sh_size == old_size) { wr64(b + sh + 0x20, code_len); text_shndx = (int64_t)s; }
        else if (sh_offset > start) wr64(b + sh + 0x18, moved(sh_offset));
    }
    if (text_shndx >= 0)
        for (uint64_t s = 0; s < shnum; ++s) {
            if (!inside(shoff, 64) || s > (n - shoff - 64) / 64) break;
            const uint64_t sh = shoff + s * 64;
            if (rd32(b + sh + 4) != SHT_SYMTAB) continue;
            const uint64_t sym_off = rd64(b + sh + 0x18), sym_total = rd64(b + sh + 0x20);
            if (sym_total >= 24 && sym_off > n) throw std::runtime_error("failed to parse ELF: symbol table offset past end of file");
            for (uint64_t i = 0; i < sym_total / 24; ++i) {
                if (!inside(sym_off, 24) || i > (n - sym_off - 24) / 24) break;
                const uint64_t so = sym_off + i * 24;
                if (rd16(b + so + 6) == (uint64_t)text_shndx && (b[so + 4] >> 4) >= 1) wr64(b + so + 16, code_len);
            }
            break;   // the first symbol table only
        }
    // The first section that starts with a DWARF64 length marker is taken to be .debug_frame.
    for (uint64_t s = 0; s < shnum; ++s) {
        if (!inside(shoff, 64) || s > (n - shoff - 64) / 64) break;
        const uint64_t sh = shoff + s * 64;
        const uint64_t sh_offset = rd64(b + sh + 0x18), sh_size = rd64(b + sh + 0x20);
        if (sh_size < 48 || sh_offset > n || sh_size > n - sh_offset) continue;
        if (rd32(b + sh_offset) != 0xFFFFFFFFu) continue;
        uint64_t pos = sh_offset;
        const uint64_t end = sh_offset + sh_size;
        while (pos + 36 <= end) {
            if (rd32(b + pos) != 0xFFFFFFFFu) break;
            const uint64_t length = rd64(b + pos + 4);
            if (rd64(b + pos + 12) != ~0ull && rd64(b + pos + 28) == old_size) wr64(b + pos + 28, code_len);
            if (length > end - pos) break;
            pos += 12 + length;
        }
        break;
    }
    return out;
}

// ---- builder -----------------------------------------------------------------------------

namespace {
struct StrTab {
    std::vector<uint8_t> data{0};
    uint32_t add(const std::string& s) {
        uint32_t off = uint32_t(data.size());
        data.insert(data.end(), s.begin(), s.end());
        data.push_back(0);
        return off;
    }
};
struct Sec {
    uint32_t name, type;
    uint64_t flags;
    const uint8_t* data;
    uint64_t size;     // file bytes (0 for NOBITS)
    uint64_t memsize;  // sh_size
    uint64_t align;
    uint32_t link, info;
    uint64_t entsize;
    uint64_t offset;
    uint64_t pad_words;  // text only: padding words appended after `data`
};
}  // namespace

// NOP and a branch-to-self, the two words the reference pads text sections with.
static const uint8_t kNop[16] = {0x18, 0x79, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0xc0, 0x0f, 0};
static const uint8_t kBraSelf[16] = {0x47, 0x79, 0xfc, 0x00, 0xfc, 0xff, 0xff, 0xff,
                                      0xff, 0xff, 0x83, 0x03, 0x00, 0xc0, 0x0f, 0x00};

uint64_t elf_build(const std::vector<BuildKernel>& kernels, uint8_t* out, uint64_t capacity) {
    const size_t n = kernels.size();
    const size_t total_sections = 9 + 4 * n;
    if (total_sections >= 0xFF00 || 3 + 2 * n > 0xFFFF) throw std::runtime_error("too many kernels for one ELF");
    const size_t base = 8;
    auto text_k = [&](size_t k) { return base + n + k; };
    auto func_sym = [&](size_t k) { return 3 + n + k; };

    StrTab shstr, str;
    const uint32_t n_shstr = shstr.add(".shstrtab"), n_str = shstr.add(".strtab"), n_sym = shstr.add(".symtab");
    const uint32_t n_tk = shstr.add(".note.nv.tkinfo"), n_cu = shstr.add(".note.nv.cuinfo");
    const uint32_t n_info = shstr.add(".nv.info"), n_compat = shstr.add(".nv.compat");
    std::vector<uint32_t> n_info_k(n), n_text_k(n), n_const_k(n), n_shared_k(n), s_func(n), s_const(n), s_shared(n);
    for (size_t k = 0; k < n; ++k) {
        n_info_k[k] = shstr.add(".nv.info." + kernels[k].name);
        n_text_k[k] = shstr.add(".text." + kernels[k].name);
        n_const_k[k] = shstr.add(".nv.constant0." + kernels[k].name);
        n_shared_k[k] = shstr.add(".nv.shared." + kernels[k].name);
    }
    const uint32_t n_shared = shstr.add(".nv.shared.reserved.0");
    for (size_t k = 0; k < n; ++k) s_func[k] = str.add(kernels[k].name);
    for (size_t k = 0; k < n; ++k) s_const[k] = str.add(".nv.constant0." + kernels[k].name);
    for (size_t k = 0; k < n; ++k) s_shared[k] = str.add(".nv.shared." + kernels[k].name);

    std::vector<uint64_t> text_size(n);
    for (size_t k = 0; k < n; ++k) {
        if (kernels[k].bytes % 16) throw std::runtime_error("kernel code must be whole 16-byte words");
        text_size[k] = (kernels[k].bytes + 127) / 128 * 128;
    }

    // Symbols: null, two note sections, N text sections, N global functions, N constant
    // banks, N shared sections.
    std::vector<uint8_t> symtab((3 + 4 * n) * 24, 0);
    auto sym = [&](size_t idx, uint32_t name, uint8_t info, uint8_t other, size_t shndx, uint64_t size) {
        uint8_t* s = &symtab[idx * 24];
        wr32(s, name); s[4] = info; s[5] = other; wr16(s + 6, uint16_t(shndx)); wr64(s + 16, size);
    };
    sym(1, 0, 3, 0, 4, 0);
    sym(2, 0, 3, 0, 5, 0);
    for (size_t k = 0; k < n; ++k) {
        sym(3 + k, 0, 3, 0, text_k(k), 0);
        sym(func_sym(k), s_func[k], 0x12, 0x10, text_k(k), text_size[k]);
        sym(3 + 2 * n + k, s_const[k], 3, 0, base + 3 * n + 1 + k, 0);
        sym(3 + 3 * n + k, s_shared[k], 3, 0, base + 2 * n + 1 + k, 0);
    }

    static const uint8_t kNote[16] = {0};
    static const uint8_t kConst0[0x380] = {0};
    std::vector<Sec> secs;
    auto add = [&](uint32_t name, uint32_t type, uint64_t flags, const uint8_t* data, uint64_t size, uint64_t align,
                   uint32_t link, uint32_t info, uint64_t entsize) {
        secs.push_back(Sec{name, type, flags, data, type == SHT_NOBITS ? 0 : size, size, align, link, info, entsize, 0, 0});
    };
    add(0, 0, 0, nullptr, 0, 1, 0, 0, 0);
    add(n_shstr, SHT_STRTAB, 0, shstr.data.data(), shstr.data.size(), 1, 0, 0, 0);
    add(n_str, SHT_STRTAB, 0, str.data.data(), str.data.size(), 1, 0, 0, 0);
    add(n_sym, SHT_SYMTAB, 0, symtab.data(), symtab.size(), 8, 2, uint32_t(3 + n), 24);
    add(n_tk, SHT_NOTE, 0, kNote, sizeof kNote, 4, 0, 0, 0);
    add(n_cu, SHT_NOTE, 0, kNote, sizeof kNote, 4, 4, 7, 0);
    add(n_info, 0x70000000u, 0, kNote, 0, 4, 3, 0, 0);
    add(n_compat, 0x70000086u, 0, kNote, sizeof kNote, 4, 0, 0, 0);
    for (size_t k = 0; k < n; ++k) add(n_info_k[k], 0x70000000u, 0x40, kNote, 0, 4, 3, uint32_t(text_k(k)), 0);
    for (size_t k = 0; k < n; ++k) {
        add(n_text_k[k], SHT_PROGBITS, 0x6, kernels[k].code, kernels[k].bytes, 128, 3, uint32_t(func_sym(k)), 0);
        secs.back().pad_words = (text_size[k] - kernels[k].bytes) / 16;
        secs.back().memsize = secs.back().size = text_size[k];
    }
    add(n_shared, SHT_NOBITS, 0x3, nullptr, 0x40, 1, 0, 0, 0);
    for (size_t k = 0; k < n; ++k) add(n_shared_k[k], SHT_NOBITS, 0x43, nullptr, 0x40, 4, 0, uint32_t(text_k(k)), 0);
    for (size_t k = 0; k < n; ++k) add(n_const_k[k], SHT_PROGBITS, 0x42, kConst0, sizeof kConst0, 4, 0, uint32_t(text_k(k)), 0);
    if (secs.size() != total_sections) throw std::runtime_error("internal: section count");

    const uint64_t n_phdrs = 3 + 2 * n;
    uint64_t off = 64 + n_phdrs * 56;
    off = (off + 3) & ~3ull;
    for (size_t i = 1; i < secs.size(); ++i) {
        Sec& s = secs[i];
        if (s.type == SHT_NOBITS) { s.offset = off; continue; }
        if (s.align > 1) off = (off + s.align - 1) / s.align * s.align;
        s.offset = off;
        off += s.size;
    }
    off = (off + 7) & ~7ull;
    const uint64_t sh_off = off, total = sh_off + 64 * total_sections;
    if (!out) return total;
    if (capacity < total) throw std::runtime_error("output buffer too small for the ELF");
    memset(out, 0, 64 + n_phdrs * 56);

    // ELF header.
    memcpy(out, "\x7f" "ELF", 4);
    out[4] = 2; out[5] = 1; out[6] = 1; out[7] = 0x33; out[8] = 7;
    wr16(out + 0x10, 2); wr16(out + 0x12, 190); wr32(out + 0x14, 1);
    wr64(out + 0x20, 64); wr64(out + 0x28, sh_off); wr32(out + 0x30, 0x06007802u);
    wr16(out + 0x34, 64); wr16(out + 0x36, 56); wr16(out + 0x38, uint16_t(n_phdrs));
    wr16(out + 0x3A, 64); wr16(out + 0x3C, uint16_t(total_sections)); wr16(out + 0x3E, 1);

    // Section contents.
    uint64_t cursor = 64 + n_phdrs * 56;
    for (size_t i = 1; i < secs.size(); ++i) {
        const Sec& s = secs[i];
        if (s.type == SHT_NOBITS || s.size == 0) continue;
        memset(out + cursor, 0, size_t(s.offset - cursor));
        const uint64_t code_bytes = s.size - 16 * s.pad_words;
        memcpy(out + s.offset, s.data, size_t(code_bytes));
        for (uint64_t w = 0; w < s.pad_words; ++w)
            memcpy(out + s.offset + code_bytes + 16 * w, w + 1 == s.pad_words ? kBraSelf : kNop, 16);
        cursor = s.offset + s.size;
    }
    memset(out + cursor, 0, size_t(sh_off - cursor));

    // Section headers.
    for (size_t i = 0; i < secs.size(); ++i) {
        const Sec& s = secs[i];
        uint8_t* h = out + sh_off + 64 * i;
        memset(h, 0, 64);
        wr32(h, s.name); wr32(h + 4, s.type); wr64(h + 8, s.flags);
        wr64(h + 0x18, s.offset); wr64(h + 0x20, s.type == SHT_NOBITS ? s.memsize : s.size);
        wr32(h + 0x28, s.link); wr32(h + 0x2C, s.info); wr64(h + 0x30, s.align); wr64(h + 0x38, s.entsize);
    }

    // Program headers: PHDR, one LOAD per text section, notes, shared (NOBITS), one per constant bank.
    size_t ph = 0;
    auto phdr = [&](uint32_t type, uint32_t flags, uint64_t offset, uint64_t filesz, uint64_t memsz) {
        uint8_t* p = out + 64 + 56 * ph++;
        wr32(p, type); wr32(p + 4, flags); wr64(p + 8, offset); wr64(p + 0x20, filesz); wr64(p + 0x28, memsz);
        wr64(p + 0x30, 8);
    };
    phdr(6, 4, 64, n_phdrs * 56, n_phdrs * 56);
    for (size_t k = 0; k < n; ++k) phdr(1, 5, secs[text_k(k)].offset, text_size[k], text_size[k]);
    phdr(1, 4, secs[4].offset, secs[7].offset + secs[7].size - secs[4].offset, secs[7].offset + secs[7].size - secs[4].offset);
    phdr(1, 6, secs[base + 2 * n].offset, 0, 0x40);
    for (size_t k = 0; k < n; ++k) phdr(1, 4, secs[base + 3 * n + 1 + k].offset, sizeof kConst0, sizeof kConst0);
    return total;
}

}  // namespace cubit
