"""SASS text layer: parser, lowering to (record, patch), and text -> word known answers.

Expected values are the reference's own (tests/encoding.rs of kacper-daftcode/cubit; the line
of each is cited).  The CPU tests turn a lowered record into a word with the CPU oracle's
record-level encode and apply the patch; the GPU tests go through cubit_text_encode, i.e. the
batch encode kernel.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import cubit_b200

GOLDEN = json.loads((Path(__file__).parent / "golden" / "encoding_words.json").read_text())
SCHED_MASK = 0x1FFFF << 105
TEXT_CASES = [c for c in GOLDEN["cases"] if c["kind"] in ("clean128", "lo64")]


@pytest.fixture(scope="module")
def host_codec():
    return cubit_b200.Codec(devices=())


def to_int(row) -> int:
    return int.from_bytes(np.asarray(row, np.uint8).tobytes(), "little")


def cpu_encode(codec, oracle, text, addr=0, program=False):
    """Words of `text` without a GPU: lower, oracle record encode, patch."""
    form, slots, ctrl, clear, set_ = codec.lower_text(text, addr, program=program)
    if len(form) == 0:
        return []
    words = oracle.encode_batch(form, np.ascontiguousarray(slots), ctrl)
    return [(to_int(words[i]) & ~to_int(clear[i])) | to_int(set_[i]) for i in range(len(form))]


# ---- parser (reference tests/encoding.rs:87-145 and src/parser.rs) -------------------------

def test_parser_operands(host_codec):
    p = host_codec.parse_text("IADD3 R5, PT, PT, R9, R4, R5 ;")
    assert p["key"] == "IADD3_R_P_P_R_R_R" and len(p["operands"]) == 6 and p["opcode"] == "IADD3"    # :89-92
    assert p["guard"] is None
    p = host_codec.parse_text("@P0 IADD3 R5, PT, PT, R9, R4, R5 ;")
    assert p["guard"] == {"pred": 0, "negated": False, "uniform": False}                              # :98-101
    p = host_codec.parse_text("@!P1 BRA 0x100 ;")
    assert p["guard"]["pred"] == 1 and p["guard"]["negated"]                                          # :106-109
    p = host_codec.parse_text("DADD R2, R18, 1 ;")
    assert p["key"] == "DADD_R_R_FI" and p["operands"][2]["kind"] == "FloatImm"                       # :114-120
    assert p["operands"][2]["bits"] == 0x3FF0000000000000
    p = host_codec.parse_text("LDG.E R10, desc[UR4][R2.64+0x8] ;")
    d = p["operands"][1]
    assert p["key"] == "LDG_R_dARI" and (d["ur_idx"], d["base_reg"], d["offset"]) == (4, 2, 8)         # :125-133
    assert d["base_reg_suffix"] == "64" and p["mod_group"] == "E"
    p = host_codec.parse_text("BSSY B7, 0x100 ;")
    assert p["key"] == "BSSY_B_II" and p["operands"][0] == {"type": "B", "kind": "Barrier", "num": 7}  # :139-144
    p = host_codec.parse_text("IADD3 R0, PT, PT, R5, -0x20, R7 ;")
    assert p["key"] == "IADD3_R_P_P_R_II_R" and p["operands"][4]["value"] == -0x20                    # :32-33


def test_parser_operand_forms(host_codec):
    P = host_codec.parse_text
    ops = P("FFMA R1, -|R2|.reuse, ~R3, -RZ")["operands"]
    assert ops[1] == {"type": "R", "kind": "Reg", "num": 2, "neg": True, "abs": True, "inv": False, "reuse": True}
    assert ops[2]["inv"] and ops[3]["num"] == 255 and ops[3]["neg"]
    ops = P("MOV R1, c[0x3][R4+0x10]")["operands"]
    assert ops[1] == {"type": "cARI", "kind": "ConstMem", "base_reg": 4, "ur_reg": None, "bank": 3, "offset": 16}
    assert P("LDC R1, c[0x0][0x37c]")["key"] == "LDC_R_cAI"
    assert P("LDS R1, [R2+UR5+-0x8]")["operands"][1]["offset"] == -8
    assert P("LDS R1, [UR5+0x8]")["key"] == "LDS_R_AURI" and P("LDS R1, [0x8]")["key"] == "LDS_R_AI"
    assert P("LDG.E R1, desc[URZ][R2.64]")["operands"][1]["ur_idx"] == 63
    assert P("UMOV UR4, URZ")["operands"][1] == {"type": "UR", "kind": "UReg", "num": 63, "neg": False, "reuse": False,
                                                   "is_zero": True}
    assert P("ISETP.GE.AND P0, PT, R1, 0x7F7F7F7F, !UP3")["operands"][3]["value"] == 0x7F7F7F7F
    assert P("ISETP.GE.AND P0, PT, R1, 0x7F7F7F7F, !UP3")["operands"][4] == {"type": "UP", "kind": "UPred", "num": 3,
                                                                               "neg": True}
    # 0x + exactly eight hex digits + F is a raw f32 pattern; INF / NAN; decimal point -> float.
    assert P("FADD R1, R2, 0x3f800000F")["operands"][2]["bits"] == 0x3FF0000000000000
    assert P("FADD R1, R2, -INF")["operands"][2]["bits"] == 0xFFF0000000000000
    assert P("MOV R1, 1.5")["operands"][1]["kind"] == "FloatImm" and P("MOV R1, 15")["operands"][1]["kind"] == "Imm32"
    assert P("S2R R1, SR_TID.X")["operands"][1] == {"type": "L", "kind": "SysReg", "text": "SR_TID.X"}
    assert P("DEPBAR.LE SB0, 0x1")["key"] == "DEPBAR_II_II" and P("BRA loop_end")["operands"][0]["kind"] == "Label"
    # branch opcodes: "register target" separated by a space only
    assert P("BRX R20 0x60")["key"] == "BRX_R_II" and P("BRX R20 -0x60")["operands"][1]["value"] == -0x60
    # annotations after '?' / '&' are dropped, opaque ".?n" parts leave an empty modifier
    p = P("ISETP.EQ.AND.?6.?0 P0, PT, R1, R2, PT &req={0} ?WAIT1")
    assert p["opcode_full"] == "ISETP.EQ.AND." and p["key"] == "ISETP_P_P_R_R_P" and p["mod_group"] == "AND,EQ"


def test_parser_errors_and_control_codes(host_codec):
    with pytest.raises(ValueError, match=r'parse error: unrecognized SASS: "\[R1\]"'):
        host_codec.parse_text("[R1]")
    with pytest.raises(ValueError, match="parse error: invalid control code string"):
        host_codec.parse_text("[B------:R-:W-:-:S1] NOP")
    for s in GOLDEN["ctrl_strings"] + ["B012345:R5:W0:Y:S15"]:                      # scheduling.rs:119-133, encoding.rs:148-158
        p = host_codec.parse_text(f"[{s}] IADD3 R5, PT, PT, R9, R4, R5 ;")
        assert p["ctrl"] == s and p["hand_sched"]
    assert host_codec.parse_text("NOP")["ctrl"] == "B------:R-:W-:-:S01"


# ---- text -> word known answers -----------------------------------------------------------

@pytest.mark.parametrize("case", TEXT_CASES, ids=[c["source"].split(":")[1] for c in TEXT_CASES])
def test_golden_text_words_cpu(host_codec, oracle, case):
    w = cpu_encode(host_codec, oracle, case["sass"])[0]
    exp = int(case["word"], 16)
    if case["kind"] == "lo64":
        assert w & (2**64 - 1) == exp, case["source"]
    else:
        assert w & ~SCHED_MASK == exp & ~SCHED_MASK, case["source"]
    if "key" in case:   # the variant the text selects is the one the case names
        form = host_codec.lower_text(case["sass"], 0, program=False)[0]
        m = host_codec.variant(int(form[0]))
        assert (m.key, m.mod_group) == (case["key"], case["mod_group"])


def test_partial_field_answers_cpu(host_codec, oracle):
    enc = lambda s: cpu_encode(host_codec, oracle, s)[0]
    lo = enc("IADD3 R0, PT, PT, R5, -0x20, R7 ;") & (2**64 - 1)
    assert (lo >> 32) & 0xFFFFFFFF == 0xFFFFFFE0 and lo & 0xFFFF == 0x7810          # encoding.rs:36-37
    assert (enc("HADD2.F32 R42, -RZ, R5.H0_H0 ;") >> 32) & 0xFF == 5                # :53
    assert (enc("HADD2.F32 R42, -RZ, R41.H0_H0 ;") >> 32) & 0xFF == 41              # :54
    with_ = enc("LDG.E.U16 R56, desc[UR4][R26.64+0x400] ;") & (2**64 - 1)
    without = enc("LDG.E.U16 R56, desc[UR4][R26.64] ;") & (2**64 - 1)
    assert with_ - without == 0x400 << 40                                            # :83
    assert enc("IADD3 R5, PT, PT, R9, R4, R5 ;") != 0                                # :21
    assert enc("IMAD.WIDE R8, R31, R6, R8 ;") & 0xFFFF == 0x7225                     # :319
    # default control code B------:R-:W-:-:S01 lands in bits 121:105
    assert (enc("IADD3 R5, PT, PT, R9, R4, R5 ;") >> 105) & 0x1FFFF == (7 << 8) | (7 << 5) | 1


def test_real_table_refusals_and_wildcard(host_codec):
    with pytest.raises(ValueError) as e:                                             # encoding.rs:524-533
        host_codec.lower_text("IMNMX.U32 R7, R7, 0xf, PT ;", 0, program=False)
    msg = str(e.value)
    assert msg.startswith("encode error: no operand-compatible table entry; attempted keys: [")
    assert "IMNMX.U32_R_R_II_P" in msg and "IMNMX_R_R_II_P" in msg and "not in table" in msg
    form = host_codec.lower_text("F2FP.SATFINITE.E4M3.F32.PACK_AB_MERGE_C R26, R14, R26 ;", 0, program=False)[0]
    assert len(form) == 1                                                            # :536-544


def synthetic_table(tmp_path, key, group, and_base, fields):
    table = {key: {"mod_groups": {group: {"and_base": hex(and_base), "variable_mask": "0x0", "fields": [
        {"shift": s, "bits": b, "token_idx": t, "extraction": e} for s, b, t, e in fields]}}}}
    path = tmp_path / f"{key}.json"
    path.write_text(json.dumps(table))
    return cubit_b200.Codec(devices=(), table_path=path)


def test_rejects_entries_that_do_not_fit_the_operands(tmp_path):
    # register-form fields under an immediate-form key (encoding.rs:439-467)
    c = synthetic_table(tmp_path, "ISETP_P_P_R_II_P", "AND,LT", 0x720C, [(24, 8, 3, "reg"), (32, 8, 4, "reg"), (81, 3, 1, "pred")])
    with pytest.raises(ValueError) as e:
        c.lower_text("ISETP.LT.AND P1, PT, R2, 0x1c0, PT ;", 0, program=False)
    msg = str(e.value)
    assert "attempted keys" in msg and "ISETP_P_P_R_II_P" in msg and "REJECTED" in msg
    assert "field (shift=32 ext=Reg) expects a different operand kind than operand 4 (II)" in msg
    # immediate-form field under a register-form key; RZ still goes through it (encoding.rs:470-497)
    c = synthetic_table(tmp_path, "VIMNMX_R_R_R_P", "U32", 0x7848, [(16, 8, 1, "reg"), (24, 8, 2, "reg"), (32, 32, 3, "imm")])
    with pytest.raises(ValueError, match="REJECTED"):
        c.lower_text("VIMNMX.U32 R4, R4, R5, PT ;", 0, program=False)
    assert len(c.lower_text("VIMNMX.U32 R4, R4, RZ, PT ;", 0, program=False)[0]) == 1
    # registers frozen in and_base (encoding.rs:500-521)
    c = synthetic_table(tmp_path, "FSETP_P_P_R_R_P", "AND,GT", 0x0400000003F24000000000040500720B, [(123, 1, 4, "reuse")])
    with pytest.raises(ValueError, match=r"operand 1 \(P2\) has no field able to encode it"):
        c.lower_text("FSETP.GT.AND P2, PT, R8, RZ, PT ;", 0, program=False)


# ---- programs: labels, comments, control prefixes, raw words --------------------------------

def test_program_labels_and_prefixes_cpu(host_codec, oracle):
    program = """
        // a comment ; with a semicolon
        start:
        /*0000*/ [B--2---:R0:W1:-:S07] IADD3 R5, PT, PT, R9, R4, R5 ;   # trailing
        BRA end ; NOP
        .section ignored_as_in_the_reference
        back: BRA start
        __raw__0x000fc00000000000000000000000794d ;
        end: EXIT
    """
    # ".section ..." parses as an instruction in the reference too and then fails to encode
    with pytest.raises(ValueError, match=r"encode error at addr 0x130: no operand-compatible"):
        host_codec.lower_text(program, 0x100, program=True)
    program = program.replace(".section ignored_as_in_the_reference", "")
    words = cpu_encode(host_codec, oracle, program, 0x100, program=True)
    assert len(words) == 6
    one = lambda s, a: cpu_encode(host_codec, oracle, s, a)[0]
    assert (words[0] >> 105) & 0x1FFFF == (0b000100 << 11) | (0 << 8) | (1 << 5) | 7          # B--2---:R0:W1:-:S07
    assert words[0] & ~SCHED_MASK == one("IADD3 R5, PT, PT, R9, R4, R5", 0x100) & ~SCHED_MASK
    assert words[1] == one("BRA 0x150", 0x110)         # "end" is the sixth statement: 0x100 + 5 * 16
    assert words[2] == one("NOP", 0x120)
    assert words[3] == one("BRA 0x100", 0x130)         # backward branch, sign-extended
    assert (words[3] >> 64) & 0x3FFFF == 0x3FFFF
    assert words[4] == 0x000FC00000000000000000000000794D
    assert words[5] == one("EXIT", 0x150)
    # the self-branch padding word of the reference's cubin builder is "BRA <own address>"
    pad = {p["name"]: int(p["word"], 16) for p in GOLDEN["padding_words"]}
    assert one("BRA 0x40", 0x40) & ~SCHED_MASK == pad["bra_self"] & ~SCHED_MASK
    assert one("NOP", 0) & ~SCHED_MASK == pad["nop"] & ~SCHED_MASK


# ---- through the GPU ------------------------------------------------------------------------

@pytest.mark.gpu
def test_text_encode_gpu(codec, oracle):
    for case in TEXT_CASES:
        lo, hi = codec.encode(case["sass"])
        w = lo | (hi << 64)
        exp = int(case["word"], 16)
        if case["kind"] == "lo64":
            assert lo == exp, case["source"]
        else:
            assert w & ~SCHED_MASK == exp & ~SCHED_MASK, case["source"]
        assert w == cpu_encode(codec, oracle, case["sass"])[0]
        if "key" in case:                    # and the word decodes back to the variant the text names
            d = codec.decode(lo, hi)
            assert (d["key"], d["mod_group"]) == (case["key"], case["mod_group"])
    with pytest.raises(ValueError, match="encode error: no operand-compatible table entry"):
        codec.encode("IMNMX.U32 R7, R7, 0xf, PT ;")
    with pytest.raises(ValueError, match="parse error: unrecognized SASS"):
        codec.encode("[R1]")


@pytest.mark.gpu
def test_text_program_gpu(codec, oracle):
    lines = [c["sass"] for c in TEXT_CASES] * 50 + ["top: BRA top", "__raw__0x0123456789abcdef0123456789abcdef"]
    program = "\n".join(lines)
    words = codec.encode_text(program, 0x1000, program=True)
    assert words.shape == (len(lines), 16)
    expect = cpu_encode(codec, oracle, program, 0x1000, program=True)
    assert [to_int(w) for w in words] == expect
    data, count = cubit_b200.encode_lines("BRA end; NOP; end: EXIT")
    assert count == 3 and len(data) == 48
    assert cubit_b200.encode("NOP") == codec.encode("NOP")
