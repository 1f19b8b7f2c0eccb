"""ISA table loading and compilation (host only): counts, provenance, strict errors."""
import hashlib
import json

import pytest

import cubit_b200
from cubit_b200 import Codec, CubitError
from cubit_b200.codec import NOT_STORED

TABLE = cubit_b200.build.PKG / "tables" / "sm120.json"


def test_vendored_table_is_the_reference_table(golden):
    assert hashlib.sha256(TABLE.read_bytes()).hexdigest() == golden["table_sha256"]
    src = json.loads((TABLE.parent / "SM120_SOURCE.json").read_text())
    assert src["sha256"] == golden["table_sha256"]


def test_table_info(host_codec, oracle, golden):
    assert host_codec.table_info() == (golden["instruction_forms"], golden["encoding_variants"]) == (2001, 2872)
    assert oracle.table_info() == host_codec.table_info()


def test_variant_ids_are_bytewise_sorted_pairs(host_codec, oracle):
    raw = json.loads(TABLE.read_text())["instructions"]
    pairs = sorted(((k.encode(), m.encode()) for k, v in raw.items() for m in v.get("mod_groups", {})))
    assert len(pairs) == 2872
    for v in (0, 1, 17, 1178, 2000, 2871):
        m = host_codec.variant(v)
        assert (m.key.encode(), m.mod_group.encode()) == pairs[v]
        assert oracle.variant_name(v) == (m.key, m.mod_group)
        assert host_codec.find_variant(m.key, m.mod_group) == v
    with pytest.raises(CubitError):
        host_codec.variant(2872)
    with pytest.raises(CubitError):
        host_codec.find_variant("NO_SUCH_KEY", "")


def test_field_metadata_matches_json(host_codec):
    raw = json.loads(TABLE.read_text())["instructions"]
    for v in range(0, 2872, 7):
        m = host_codec.variant(v)
        fields = raw[m.key]["mod_groups"][m.mod_group]["fields"]
        assert [(f.shift, f.bits, f.token_idx) for f in m.fields] == [(f["shift"], f["bits"], f["token_idx"]) for f in fields]
        # slot layout: only bits below bit 96 are stored; layout 0 keeps fields apart, layout 1 keeps them in place
        used = 0
        for f in m.fields:
            assert f.stored_bits == max(0, min(f.shift + f.bits, 96) - f.shift)
            if not f.stored_bits:
                assert f.dst_pos == NOT_STORED
                continue
            span = ((1 << f.stored_bits) - 1) << f.dst_pos
            assert f.dst_pos + f.stored_bits <= 256
            if m.layout_kind == 0:
                assert not used & span
                assert f.dst_pos % 32 == 0 if f.stored_bits > 1 else f.dst_pos >= 224
            else:
                assert f.dst_pos == f.shift
            used |= span


def test_most_variants_get_one_slot_per_operand_field(host_codec):
    # 2,434 variants have neither overlapping stored fields nor a multi-bit field across a 32-bit limb
    # boundary; the slot-by-limb pattern of layout 0 holds 2,309 of them.
    kinds = [host_codec.variant(v).layout_kind for v in range(2872)]
    assert kinds.count(0) >= 2300 and kinds.count(1) > 0


def test_field_names_and_extraction_spellings(host_codec):
    m = host_codec.variant(host_codec.find_variant("IMAD_R_R_R_R", "WIDE"))
    assert [f.name for f in m.fields[:3]] == ["Rd", "Ra", "Rc"] and m.fields[3].name == "[122:122]"
    assert m.opcode == "IMAD"
    assert host_codec.variant(host_codec.find_variant("F2FP.F16.E4M3.UNPACK_B_R_R", "")).opcode == "F2FP.F16.E4M3.UNPACK_B"
    seen = set()
    for v in range(2872):
        seen.update(f.extraction for f in host_codec.variant(v).fields)
    assert "upred" not in seen and "" not in seen and "none" in seen
    assert {"immdec", "guardlo3", "negshl1", "bytesel", "cm16off"} <= seen or len(seen) > 30


def test_no_control_bits_baked_into_and_base():
    """Reference tests/encoding.rs:201-213."""
    raw = json.loads(TABLE.read_text())["instructions"]
    for key, v in raw.items():
        for mods, e in v.get("mod_groups", {}).items():
            assert int(e["and_base"], 16) >> 105 == 0, (key, mods)
    assert "HADD2_R_R_II" not in raw   # reference tests/encoding.rs:216-221


def flat_table(group: str) -> str:
    return '{"TEST_R":{"mod_groups":{"":' + group + "}}}"


@pytest.mark.parametrize("group,why", [
    ('{"and_base":"0x1","variable_mask":"0x100000000000000000000000000000000","fields":[]}', "wider than 128"),
    ('{"and_base":"0x1","fields":[{"shift":122,"bits":8,"token_idx":1,"extraction":"reg"}]}', "outside 128-bit"),
    ('{"and_base":"0x1","fields":[{"shift":16,"bits":8,"token_idx":1,"extraction":"mystery"}]}', "unknown extraction"),
    ('{"and_base":"0x1","fields":[{"shift":16,"bits":0,"token_idx":1,"extraction":"reg"}]}', "outside 128-bit"),
    ('{"fields":[]}', "and_base"),
])
def test_malformed_tables_are_rejected(tmp_path, oracle, group, why):
    """Reference src/table.rs:512-534: the same three rejections, plus zero-width fields and a missing base."""
    from oracle_lib import Oracle
    p = tmp_path / "bad.json"
    p.write_text(flat_table(group))
    with pytest.raises(CubitError) as e:
        Codec(devices=(), table_path=p)
    assert e.value.code == -2 and why in e.value.message
    with pytest.raises(ValueError):
        Oracle(table_path=p)


def test_flat_format_and_missing_variable_mask(tmp_path):
    p = tmp_path / "ok.json"
    p.write_text(flat_table('{"and_base":"0x7210","fields":[{"shift":16,"bits":8,"token_idx":1,"extraction":"reg"}]}'))
    c = Codec(devices=(), table_path=p)
    assert c.table_info() == (1, 1)
    assert c.variant(0).key == "TEST_R" and c.variant(0).fields[0].name == "Rd"


def test_cubit_table_env_is_strict(tmp_path, monkeypatch):
    monkeypatch.setenv("CUBIT_TABLE", str(tmp_path / "absent.json"))
    with pytest.raises(CubitError) as e:
        Codec(devices=())
    assert e.value.code == -2 and "failed to read" in e.value.message
    good = tmp_path / "one.json"
    good.write_text(flat_table('{"and_base":"0x1","fields":[]}'))
    monkeypatch.setenv("CUBIT_TABLE", str(good))
    assert Codec(devices=(), table_path=TABLE).table_info() == (1, 1)   # the variable wins over the argument


def test_the_reference_module_name_is_importable():
    """`import cubit` is what a user of the reference writes (reference src/python.rs:215-225)."""
    import cubit
    assert cubit.table_info() == (2001, 2872)
    assert sorted(cubit.__all__) == sorted(["encode", "decode", "decode_kernel", "table_info", "to_sass", "asm"])
    for name in cubit.__all__:
        assert callable(getattr(cubit, name))
    with pytest.raises(NotImplementedError):
        cubit.asm("NOP")
