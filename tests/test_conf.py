"""triton-ext.conf parsing and TRITON_EXT_NAMES gating (reference: cmake/utils.cmake:52-136)."""
import os

import pytest

from triton_ext_b200 import build, conf


def test_parse_forms():
    assert conf.parse_conf_text("loop_split;experimental\n") == conf.ExtConf("loop_split", "experimental", "", "")
    assert conf.parse_conf_text("x") .status == "experimental"  # default, utils.cmake:96
    c = conf.parse_conf_text(" name ; stable ; abc123 ")
    assert (c.name, c.status, c.hash) == ("name", "stable", "abc123")
    with pytest.raises(ValueError):
        conf.parse_conf_text("   \n")


def test_shipped_confs_match_extension_names():
    for rel, _cls, _src, _cuda in build.EXTENSIONS:
        c = conf.read_conf(os.path.join(build.CSRC, rel))
        assert c.status == "experimental"
        assert os.path.basename(c.path) == "triton-ext.conf"
    names = [conf.read_conf(os.path.join(build.CSRC, rel)).name for rel, *_ in build.EXTENSIONS]
    assert names == ["loop_split", "dot_tile_select", "b200_dot"]


def test_underscore_alias(tmp_path):
    d = tmp_path / "Ext"
    d.mkdir()
    (d / "triton_ext.conf").write_text("aliased;experimental")
    assert conf.read_conf(str(d)).name == "aliased"
    (d / "triton-ext.conf").write_text("hyphen;experimental")
    assert conf.read_conf(str(d)).name == "hyphen"  # the spelling the reference's CMake reads wins


def test_names_gating(tmp_path, monkeypatch):
    d = tmp_path / "A"
    d.mkdir()
    (d / "triton-ext.conf").write_text("alpha;experimental")
    assert conf.should_build(str(d), [])              # empty allow-list builds everything
    assert conf.should_build(str(d), ["alpha", "b"])
    assert not conf.should_build(str(d), ["beta"])
    assert not conf.should_build(str(tmp_path / "missing"), [])
    monkeypatch.setenv("TRITON_EXT_NAMES", "beta;gamma")
    assert not conf.should_build(str(d))
    monkeypatch.setenv("TRITON_EXT_NAMES", "alpha")
    assert conf.should_build(str(d))
    e = tmp_path / "B"
    e.mkdir()
    (e / "triton-ext.conf").write_text("")
    assert not conf.should_build(str(e), [])


def test_discover(tmp_path):
    for n in ("X", "Y"):
        (tmp_path / n).mkdir()
        (tmp_path / n / "triton-ext.conf").write_text(f"{n.lower()};experimental")
    (tmp_path / "Z").mkdir()
    assert [c.name for c in conf.discover(str(tmp_path))] == ["x", "y"]
