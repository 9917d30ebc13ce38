"""The synthetic engine directory on the host: the generator writes what the reference loader parses
(`engine/engine.cu:54-75`) and every address the loader derives lies inside its file
(`engine/engine.cu:166-275`); corrupted directories are reported, not loaded."""
import importlib
import os

import numpy as np
import pytest

from conftest import PKG_NAME

ed = importlib.import_module(PKG_NAME + ".engine_dir")


@pytest.fixture(scope="module")
def directory(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("engine"))
    ed.write_engine_dir(d, layers=3, dense_layers=1, vocab=1024, seed=3)
    return d


def test_index_round_trip(directory):
    ix = ed.read_index(directory)
    assert ix.cfg["num_hidden_layers"] == "3" and ix.cfg["vocab_size"] == "1024" and ix.cfg["mask_id"] == "156895"
    assert float(ix.cfg["rope_theta"]) == 3e6 and float(ix.cfg["rms_norm_eps"]) == 1e-6
    assert sorted(ix.experts) == [1, 2] and all(len(v) == 256 for v in ix.experts.values())
    t = ix.get("small.bin", "L1.router")
    assert t.dtype == "bf16" and t.shape == (256, 2048) and t.bytes == 256 * 2048 * 2
    q = ix.get("nonexpert_L0.bin", "qkv")
    assert q.off == 0 and q.bytes == ed.matrix_bytes(3072, 2048, 8) == 192 * 16 * 2096
    assert ix.get("nonexpert_L0.bin", "down").bytes == ed.matrix_bytes(2048, 5120, 8)
    assert ix.get("nonexpert_L1.bin", "down").bytes == ed.matrix_bytes(2048, 512, 8)
    with pytest.raises(KeyError):
        ix.get("small.bin", "L0.router")                 # layer 0 is the dense layer
    for f, n in ix.fsize.items():
        assert os.path.getsize(os.path.join(directory, f)) == n


def test_layout_is_loadable(directory):
    assert ed.check_layout(directory) == []


def test_experts_alias_stored_blobs(directory):
    ix = ed.read_index(directory)
    ex = ix.experts[1]
    assert {b for b, _, _ in ex} == {2, 3, 4}
    assert len({gu for _, gu, _ in ex}) == 6 and ex[0] == ex[6] == ex[252]
    size = ix.fsize["experts_L1.bin"]
    for b, gu, dn in ex:
        assert gu + ed.matrix_bytes(1024, 2048, b) <= dn and dn + ed.matrix_bytes(2048, 512, b) <= size


def test_tile_parameters_are_finite_and_centred(directory):
    ix = ed.read_index(directory)
    t = ix.get("nonexpert_L1.bin", "dense")
    raw = np.fromfile(os.path.join(directory, "nonexpert_L1.bin"), np.uint8, t.bytes, offset=t.off)
    tiles = raw.reshape(-1, ed.tile_bytes(8))
    scale = tiles[:, 2048:2080].copy().view(np.float16).astype(np.float32)
    assert np.isfinite(scale).all() and (scale > 0).all() and (tiles[:, 2080:] == 128).all()
    w = (tiles[:, :2048].astype(np.float32) - 128) * scale.mean()
    assert abs(float(w.std()) - 0.02) < 2e-3


def test_embed_is_sparse_and_reaches_the_mask_row(directory):
    p = os.path.join(directory, "embed.bin")
    assert os.path.getsize(p) == (ed.MASK_ID + 1) * 2048 * 2
    assert os.stat(p).st_blocks * 512 < 16 << 20
    e = np.memmap(p, np.float16, "r").reshape(-1, 2048)
    assert float(np.abs(e[ed.MASK_ID]).max()) > 0 and float(np.abs(e[1023]).max()) > 0
    assert float(np.abs(e[1024]).max()) == 0


def test_parser_follows_the_loader(tmp_path):
    (tmp_path / "engine.idx").write_text(
        "C a 1\nC a 2\n\nX ignored line\nT f.bin w 16 32 f32 2 4\nT f.bin w 48 32 f32 8\n"
        "E 5 2 4 100 200\nF f.bin 80\n")
    ix = ed.read_index(str(tmp_path))
    assert ix.cfg == {"a": "2"}                          # later lines win
    assert ix.get("f.bin", "w").off == 48 and ix.get("f.bin", "w").shape == (8,)
    assert ix.experts[5] == [(0, 0, 0), (0, 0, 0), (4, 100, 200)]
    assert ix.fsize == {"f.bin": 80}
    with pytest.raises(FileNotFoundError):
        ed.read_index(str(tmp_path / "nowhere"))


def test_corrupted_directories_are_reported(directory, tmp_path):
    import shutil
    d = str(tmp_path / "bad")
    shutil.copytree(directory, d)
    idx = os.path.join(d, "engine.idx")
    lines = open(idx).read().splitlines()

    def variant(edit):
        open(idx, "w").write("\n".join(edit(list(lines))) + "\n")
        return ed.check_layout(d)

    assert variant(lambda ls: ls) == []
    assert any("lm_bits" in b for b in variant(lambda ls: [x for x in ls if not x.startswith("C lm_bits")]))
    assert any("L2.router" in b for b in variant(lambda ls: [x for x in ls if " L2.router " not in x]))
    far = variant(lambda ls: [x.replace("E 2 7 ", "E 2 7 4 999999999 0 #") if x.startswith("E 2 7 ") else x for x in ls])
    assert any("layer 2 expert 7 gate_up" in b for b in far)
    odd = variant(lambda ls: [x.replace("E 1 0 4 0 ", "E 1 0 4 8 ") if x.startswith("E 1 0 ") else x for x in ls])
    assert any("layer 1 expert 0 gate_up" in b for b in odd)
    short = variant(lambda ls: [x for x in ls if not x.startswith("E 1 255 ")])
    assert any("255 expert lines" in b for b in short)
    with open(os.path.join(d, "nonexpert_L0.bin"), "r+b") as f:
        f.truncate(1 << 20)
    cut = variant(lambda ls: ls)
    assert any("nonexpert_L0.bin" in b and "file has" in b for b in cut)
