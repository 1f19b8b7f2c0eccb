"""Extracts the known-answer words of the reference's own tests into encoding_words.json.

Run where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/cubit

Source: tests/encoding.rs of kacper-daftcode/cubit.  Every hex literal is read from the line
given below (the script fails if the file no longer has a literal there), so the values are
the reference's, not retyped.  Kinds:
  clean128  text -> word with the scheduling field (bits 121:105) masked out (enc_clean)
  lo64      text -> low 64 bits only
  raw128    a raw word the reference test decodes; `key` / `opcode` is what that test asserts
`key`/`mod_group` on the text cases is the variant the SASS text names (operand kinds give
the key suffix, the sorted dot-modifiers give the group); the reference tests do not assert
it, they are listed so the decode direction has an expected value too.
Also stored: the two padding words of src/elf_builder.rs:632-635 (NOP, branch-to-self).
"""
import json
import re
import sys
from pathlib import Path

# (line, kind, sass text or None, expected key or None, expected mod_group or None)
CASES = [
    (51, "lo64", "HADD2.F32 R7, -RZ, R0.H0_H0 ;", None, None),
    (66, "lo64", "LDS.U16 R7, [R5+0x2000] ;", None, None),
    (82, "lo64", "LDG.E.U16 R56, desc[UR4][R26.64+0x400] ;", None, None),
    (224, "clean128", "HADD2 R48, R48, R61 ;", "HADD2_R_R_R", ""),
    (233, "clean128", "FMUL R5, R5, 1.5 ;", None, None),
    (234, "clean128", "FMUL.FTZ R5, R5, 1.5 ;", None, None),
    (235, "clean128", "FMUL.RM R5, R5, 1.5 ;", None, None),
    (236, "clean128", "FMUL.RP R5, R5, 1.5 ;", None, None),
    (237, "clean128", "FMUL.RZ R5, R5, 1.5 ;", None, None),
    (250, "clean128", "LDG.E.LTC128B.128 R4, desc[UR4][R2.64] ;", "LDG_R_dARI", "128,E,LTC128B"),
    (254, "clean128", "LDG.E.LTC128B.128 R8, desc[UR4][R2.64+0x110] ;", "LDG_R_dARI", "128,E,LTC128B"),
    (266, "clean128", "QMMA.SF.16832.F32.E4M3.E4M3.E8 R12, R8, R4, R12, R0, R0, UR6 ;",
     "QMMA.SF.16832.F32.E4M3.E4M3.E8_R_R_R_R_R_R_UR", ""),
    (273, "clean128", "QMMA.SF.16832.F32.E2M1.E3M2.E8 R12, R8, R4, R12, R0, R0, UR6 ;", None, None),
    (280, "clean128", "QMMA.SF.16832.F32.E4M3.E4M3.E8 R12, R8, -R4, R12, R16, R16, UR5 ;",
     "QMMA.SF.16832.F32.E4M3.E4M3.E8_R_R_R_R_R_R_UR", ""),
    (290, "raw128", "BRA.U !UP0, 0x42110", "BRA.U_UP_II", None),
    (295, "raw128", "BRA.DIV UR4, 0x49d30", "BRA.DIV_UR_II", None),
    (318, "clean128", "IMAD.WIDE R8, R31, R6, R8 ;", "IMAD_R_R_R_R", "WIDE"),
    (329, "clean128", "SHF.L.U64.HI R7, R6, 0x1, R7 ;", None, None),
    (339, "clean128", "LDG.E.U8.CONSTANT R36, desc[UR6][R36.64+0x9000] ;", None, None),
    (348, "clean128", "FSETP.GEU.AND P0, PT, R33, -126, PT ;", None, None),
    (357, "clean128", "PLOP3.LUT P0, PT, PT, PT, PT, 0x80, 0x8 ;", "PLOP3_P_P_P_P_P_II_II", "LUT"),
    (367, "clean128", "UISETP.GE.AND UP0, UPT, UR5, 0x10, UPT ;", None, None),
    (377, "clean128", "S2R R13, SR_SWINHI ;", None, None),
    (379, "clean128", "UVIMNMX.S32 UR4, UR5, 0x40, UPT ;", None, None),
    (381, "clean128", "UVIMNMX.S32 UR4, UR10, 0x1, !UPT ;", None, None),
    (383, "clean128", "@!P0 LDGSTS.E.128 [R3], desc[UR14][R22.64] ;", None, None),
    (385, "clean128", "LDGDEPBAR ;", "LDGDEPBAR", ""),
    (387, "clean128", "DEPBAR.LE SB0, 0x1 ;", None, None),
    (395, "clean128", "LDGSTS.E [R9+0x10], desc[UR6][R6.64+-0x800] ;", None, None),
    (397, "clean128", "LDGSTS.E.64 [R9+0x20], desc[UR6][R4.64+0x400] ;", None, None),
    (399, "clean128", "LDGSTS.E.BYPASS.128 [R9+0x40], desc[UR6][R4.64+0x100] ;", None, None),
    (401, "clean128", "LDGSTS.E.LTC128B [R7+0x10], desc[UR6][R4.64+0x100] ;", None, None),
    (403, "clean128", "LDGSTS.E.128.ZFILL [R7+0x70], desc[UR6][R4.64+0x708] ;", None, None),
    (407, "clean128", "DEPBAR.LE SB0, 0x2 ;", None, None),
    (410, "clean128", "LDS.128 R16, [R0+UR5+0x800] ;", None, None),
    (412, "clean128", "STS.U16 [R20+UR13+0x4008], R129 ;", None, None),
    (414, "clean128", "FSEL R12, R3, RZ, P3 ;", "FSEL_R_R_R_P", ""),
    (425, "raw128", "F2FP.F16.E4M3.UNPACK_B R7, R8", None, None),
    (603, "lo64", "UISETP.NE.AND UP0, UPT, UR5, URZ, UPT ;", None, None),
]
RAW_OPCODE = {425: "F2FP.F16.E4M3.UNPACK_B"}
HEX = re.compile(r"0x([0-9a-fA-F_]{12,40})")


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    lines = (ref / "tests" / "encoding.rs").read_text().splitlines()
    cases = []
    for line, kind, sass, key, group in CASES:
        m = HEX.search(lines[line - 1])
        if not m:
            raise SystemExit(f"tests/encoding.rs:{line} holds no hex literal any more")
        digits = m.group(1).replace("_u128", "").replace("_", "")
        case = {"source": f"tests/encoding.rs:{line}", "kind": kind, "sass": sass, "word": "0x" + digits.lower()}
        if key is not None:
            case["key"] = key
        if group is not None:
            case["mod_group"] = group
        if line in RAW_OPCODE:
            case["opcode"] = RAW_OPCODE[line]
        cases.append(case)
    # Padding words of the cubin builder, as byte arrays in src/elf_builder.rs:632-635.
    src = (ref / "src" / "elf_builder.rs").read_text().splitlines()
    pad = []
    for first, name, key in ((632, "nop", "NOP"), (634, "bra_self", "BRA_II")):
        text = src[first - 1] + src[first]
        bytes_ = [int(b, 16) for b in re.findall(r"0x([0-9a-fA-F]{2})", text)]
        if len(bytes_) != 16:
            raise SystemExit(f"src/elf_builder.rs:{first} does not hold a 16-byte array any more")
        pad.append({"source": f"src/elf_builder.rs:{first}", "name": name, "key": key,
                    "word": "0x%032x" % int.from_bytes(bytes(bytes_), "little")})
    # Key splitting vectors of the printer's own unit tests (src/printer.rs:1414-1440): for each test the key is on
    # the first line given, the expected opcode on the next and the operand kinds on the one after.
    prn = (ref / "src" / "printer.rs").read_text().splitlines()
    printer_keys = []
    for first in (1416, 1423, 1430, 1437):
        key = re.search(r'parse_ins_key\("([^"]+)"\)', prn[first - 1])
        op = re.search(r'assert_eq!\(op, "([^"]+)"\)', prn[first])
        ops = re.findall(r'"([^"]+)"', prn[first + 1])
        if not key or not op or not ops:
            raise SystemExit(f"src/printer.rs:{first} no longer holds a parse_ins_key test")
        printer_keys.append({"source": f"src/printer.rs:{first}", "key": key.group(1), "opcode": op.group(1), "operands": ops})
    table = json.loads((ref / "tables" / "SM120_SOURCE.json").read_text())
    out = {"reference": "kacper-daftcode/cubit", "table_sha256": table["sha256"],
           "instruction_forms": table["instruction_forms"], "encoding_variants": table["encoding_variants"],
           "sched_mask": "0x%032x" % (0x1FFFF << 105), "cases": cases, "padding_words": pad, "printer_keys": printer_keys,
           "ctrl_strings": ["B--2---:R0:W1:-:S07", "B01--4-:R-:W-:-:S05", "B------:R-:W-:-:S01", "B0----5:R0:W5:Y:S05"]}
    dest = Path(__file__).with_name("encoding_words.json")
    dest.write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {dest} ({len(cases)} cases)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/cubit")
    main(sys.argv[1])
