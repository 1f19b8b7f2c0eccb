// Cubin (ELF64) text-section reader and synthetic multi-kernel builder.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace cubit {

struct TextSection {
    std::string name;
    uint64_t offset, size;
};

// Throws std::runtime_error for anything that is not a well-formed little-endian ELF64.
std::vector<TextSection> elf_text_sections(const uint8_t* bytes, uint64_t len);

struct ElfSection {
    std::string name;
    uint32_t type;
    uint64_t offset, size;   // sh_offset, sh_size
};
// Every section with a readable name, in section-header order; same errors as above.
std::vector<ElfSection> elf_sections(const uint8_t* bytes, uint64_t len);

// Replaces the bytes of text section `index` (an index into elf_text_sections) by `code`.
// Same length: copied in place.  Different length: the file is spliced and every offset
// behind the splice point is moved -- e_shoff, e_phoff, program header offsets (the segment
// holding the section grows or shrinks), section header offsets, the section's own size, the
// st_size of symbols defined in it, and a DWARF64 .debug_frame FDE range equal to the old size
// (reference src/elf.rs:71-219).  Throws std::runtime_error on a bad index or a section that
// does not lie inside the file.
std::vector<uint8_t> elf_patch_text(const uint8_t* bytes, uint64_t len, uint32_t index, const uint8_t* code,
                                    uint64_t code_len);

struct BuildKernel {
    std::string name;
    const uint8_t* code;
    uint64_t bytes;   // multiple of 16
};
// Writes the ELF into `out` (or only sizes it when out == nullptr); returns its length.
uint64_t elf_build(const std::vector<BuildKernel>& kernels, uint8_t* out, uint64_t capacity);

}  // namespace cubit
