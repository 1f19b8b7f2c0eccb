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

struct BuildKernel {
    std::string name;
    const uint8_t* code;
    uint64_t bytes;   // multiple of 16
};
// Writes the ELF into `out` (or only sizes it when out == nullptr); returns its length.
uint64_t elf_build(const std::vector<BuildKernel>& kernels, uint8_t* out, uint64_t capacity);

}  // namespace cubit
