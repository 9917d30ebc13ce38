"""A synthetic engine directory: the on-disk weight layout the reference engine loads, with seeded random contents.

The reference engine (`engine/engine.cu:166-290`, `Engine::load`) reads a directory of
  engine.idx            line index (`engine/engine.cu:54-75`, written by `quant/s07c_index.py`):
                          C <key> <value>                                    config scalar
                          T <file> <name> <offset> <bytes> <dtype> <dims..>  tensor inside a weight file
                          E <layer> <expert> <bits> <gu_off> <d_off>         routed expert inside experts_L<layer>.bin
                          F <file> <bytes>                                   file size
  small.bin             fp32 norm weights, bf16 routers, fp32 expert biases, the residual-rotation signs
  nonexpert_L<i>.bin    qkv [3072 x 2048], dense [2048 x 2048], gate_up [2I x 2048], down [2048 x I] as weight tiles
  experts_L<i>.bin      routed experts of an MoE layer (gate_up [1024 x 2048] + down [2048 x 512] each)
  lm_head.bin           the readout [V x 2048] as weight tiles
  embed.bin             fp16 embedding rows, memory-mapped by the host
A weight matrix [R x K] is R/16 strips of K/128 tiles; a tile is the 16 x 128 codes (`tile_code_bytes(bits)` bytes)
followed by 48 bytes of group parameters: 16 fp16 scales, 16 u8 zero points (`engine/moe_i8.cu:21-32`;
`quant/packlib.py` module docstring). The code bytes of a random matrix are random in any bit order, so the generator
writes random bytes there and meaningful scales and zero points.

No checkpoint can be downloaded where this runs; this directory is what lets the reference's whole engine, built on
the attention kernels of this package, be started, prefilled and stepped on a GPU. To keep it small the routed
experts of a layer alias a handful of stored blobs (the loader supports aliased entries, `engine/engine.cu:211-216`),
the layer count is a parameter, and embed.bin is a sparse file that only holds the rows a run can touch.

`read_index` and `check_layout` restate the loader's parsing and every address it derives from the index, so a
directory can be validated on the host before any GPU code sees it.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np

HID, NH, NKV, HD, NEXPERT = 2048, 16, 4, 128, 256       # engine/engine.cu:34
GROUP, META_BYTES = 128, 48                              # engine/moe_i8.cu:20-21
MASK_ID = 156895                                         # engine/decode.cu:233 (the decoder's own constant)
QKV_ROWS = (NH + 2 * NKV) * HD                           # 3072
INTER, MOE_INTER = 5120, 512                             # MLP widths the engine sizes its buffers for (engine/engine.cu:306)


def tile_code_bytes(bits: int) -> int:
    """Code bytes of one 16 x 128 tile (engine/moe_i8.cu:31)."""
    return {8: 2048, 5: 1024, 4: 1024, 3: 768, 2: 512}[bits]


def tile_bytes(bits: int) -> int:
    return tile_code_bytes(bits) + META_BYTES


def matrix_bytes(rows: int, k: int, bits: int) -> int:
    assert rows % 16 == 0 and k % GROUP == 0
    return (rows // 16) * (k // GROUP) * tile_bytes(bits)


def random_matrix(rng: np.random.Generator, rows: int, k: int, bits: int, std: float = 0.02) -> np.ndarray:
    """Bytes of a [rows x k] weight matrix whose dequantised entries (code - zero) * scale have about `std`."""
    strips, tiles, wb = rows // 16, k // GROUP, tile_code_bytes(bits)
    out = np.empty((strips, tiles, wb + META_BYTES), np.uint8)
    out[..., :wb] = rng.integers(0, 256, (strips, tiles, wb), dtype=np.uint8)
    levels = 1 << min(bits, 8)
    spread = np.sqrt((levels * levels - 1) / 12.0)      # std of a uniform code
    scale = (std / spread) * rng.uniform(0.75, 1.25, (strips, tiles, 16))
    out[..., wb:wb + 32] = scale.astype(np.float16).view(np.uint8).reshape(strips, tiles, 32)
    out[..., wb + 32:] = levels // 2
    return out.reshape(-1)


@dataclass
class Tensor:
    file: str
    name: str
    off: int
    bytes: int
    dtype: str
    shape: tuple


@dataclass
class Index:
    cfg: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)          # "file:name" -> Tensor
    experts: dict = field(default_factory=dict)          # layer -> list of (bits, gu_off, d_off)
    fsize: dict = field(default_factory=dict)

    def get(self, file: str, name: str) -> Tensor:
        key = f"{file}:{name}"
        if key not in self.tensors:
            raise KeyError(f"missing tensor {key}")
        return self.tensors[key]


def read_index(directory: str) -> Index:
    """Host restatement of the loader's index parser (engine/engine.cu:54-75): whitespace-separated fields, later lines
    overwrite earlier ones, an expert list grows to the highest expert number seen, unknown line kinds are skipped."""
    path = os.path.join(directory, "engine.idx")
    if not os.path.exists(path):
        raise FileNotFoundError(f"no {path}")
    ix = Index()
    with open(path) as f:
        for line in f:
            p = line.split()
            if not p:
                continue
            if p[0] == "C" and len(p) >= 3:
                ix.cfg[p[1]] = p[2]
            elif p[0] == "T" and len(p) >= 6:
                t = Tensor(p[1], p[2], int(p[3]), int(p[4]), p[5], tuple(int(d) for d in p[6:]))
                ix.tensors[f"{t.file}:{t.name}"] = t
            elif p[0] == "E" and len(p) >= 6:
                layer, e = int(p[1]), int(p[2])
                v = ix.experts.setdefault(layer, [])
                while len(v) <= e:
                    v.append((0, 0, 0))
                v[e] = (int(p[3]), int(p[4]), int(p[5]))
            elif p[0] == "F" and len(p) >= 3:
                ix.fsize[p[1]] = int(p[2])
    return ix


class _Writer:
    """Appends tensors to one weight file at 256-byte aligned offsets and records their index lines."""

    def __init__(self, directory: str, name: str, lines: list):
        self.name, self.lines, self.off = name, lines, 0
        self.f = open(os.path.join(directory, name), "wb")

    def add(self, tname: str, arr: np.ndarray, dtype: str, shape) -> int:
        pad = -self.off % 256
        self.f.write(b"\0" * pad)
        self.off += pad
        b = np.ascontiguousarray(arr).tobytes()
        self.lines.append(f"T {self.name} {tname} {self.off} {len(b)} {dtype} " + " ".join(str(s) for s in shape))
        self.f.write(b)
        at, self.off = self.off, self.off + len(b)
        return at

    def close(self) -> int:
        self.f.close()
        self.lines.append(f"F {self.name} {self.off}")
        return self.off


def write_engine_dir(directory: str, layers: int = 3, dense_layers: int = 1, vocab: int = 4096, seed: int = 0,
                     nonexpert_bits: int = 8, lm_bits: int = 8, expert_bits=(4, 3, 2, 4, 3, 2)) -> Index:
    """Write a directory `Engine::load` accepts. `layers` transformer layers, the first `dense_layers` with the dense
    MLP (`first_k_dense_replace`), the rest MoE layers whose 256 routed experts alias `len(expert_bits)` stored blobs
    (expert e -> blob e % len, at that blob's bit width). `vocab` rows in the readout; embed.bin is sized to hold the
    decoder's mask token row whatever `vocab` is, and holds random rows for ids < vocab and for the mask token."""
    assert vocab % 128 == 0 and 0 < dense_layers <= layers and all(b in (2, 3, 4) for b in expert_bits)
    os.makedirs(directory, exist_ok=True)
    rng = np.random.default_rng(seed)
    lines = [f"C {k} {v}" for k, v in (
        ("num_hidden_layers", layers), ("vocab_size", vocab), ("hidden_size", HID), ("num_attention_heads", NH),
        ("num_key_value_heads", NKV), ("head_dim", HD), ("num_experts", NEXPERT), ("num_experts_per_tok", 8),
        ("rms_norm_eps", 1e-06), ("rope_theta", 3000000.0), ("routed_scaling_factor", 2.5),
        ("first_k_dense_replace", dense_layers), ("intermediate_size", INTER),
        ("moe_intermediate_size", MOE_INTER), ("mask_id", MASK_ID), ("nonexpert_bits", nonexpert_bits),
        ("lm_bits", lm_bits))]

    small = _Writer(directory, "small.bin", lines)
    ones = lambda n: (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)   # noqa: E731
    for li in range(layers):
        small.add(f"L{li}.input_layernorm.weight", ones(HID), "f32", (HID,))
        small.add(f"L{li}.post_attention_layernorm.weight", ones(HID), "f32", (HID,))
        small.add(f"L{li}.attention.query_layernorm.weight", ones(HD), "f32", (HD,))
        small.add(f"L{li}.attention.key_layernorm.weight", ones(HD), "f32", (HD,))
        if li >= dense_layers:
            r = (0.02 * rng.standard_normal((NEXPERT, HID))).astype(np.float32)
            bf16 = ((r.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
            small.add(f"L{li}.router", bf16, "bf16", (NEXPERT, HID))
            small.add(f"L{li}.expert_bias", np.zeros(NEXPERT, np.float32), "f32", (NEXPERT,))
    small.add("final_norm", ones(HID), "f32", (HID,))
    small.add("signs", rng.choice(np.array([-1.0, 1.0], np.float32), HID), "f32", (HID,))
    small.close()

    for li in range(layers):
        inter = INTER if li < dense_layers else MOE_INTER
        w = _Writer(directory, f"nonexpert_L{li}.bin", lines)
        for name, rows, k in (("qkv", QKV_ROWS, HID), ("dense", HID, HID), ("gate_up", 2 * inter, HID),
                              ("down", HID, inter)):
            w.add(name, random_matrix(rng, rows, k, nonexpert_bits), f"i8tiles{nonexpert_bits}", (rows, k))
        w.close()
        if li >= dense_layers:
            x = _Writer(directory, f"experts_L{li}.bin", [])
            blobs = []
            for b in expert_bits:
                gu = x.add("gu", random_matrix(rng, 2 * MOE_INTER, HID, b), "", ())
                dn = x.add("d", random_matrix(rng, HID, MOE_INTER, b), "", ())
                blobs.append((b, gu, dn))
            lines.append(f"F experts_L{li}.bin {x.close()}")
            for e in range(NEXPERT):
                b, gu, dn = blobs[e % len(blobs)]
                lines.append(f"E {li} {e} {b} {gu} {dn}")

    lm = _Writer(directory, "lm_head.bin", lines)
    lm.lines.append(f"T lm_head.bin lm_head 0 {matrix_bytes(vocab, HID, lm_bits)} i8tiles{lm_bits} {vocab} {HID}")
    for r0 in range(0, vocab, 4096):                     # strips are independent: write in row chunks
        chunk = random_matrix(rng, min(4096, vocab - r0), HID, lm_bits)
        lm.f.write(chunk.tobytes())
        lm.off += len(chunk)
    lm.close()

    rows_total = max(vocab, MASK_ID + 1)
    with open(os.path.join(directory, "embed.bin"), "wb") as f:
        f.truncate(rows_total * HID * 2)                 # sparse: untouched rows read as zeros
        f.seek(0)
        for r0 in range(0, vocab, 8192):
            n = min(8192, vocab - r0)
            f.write((0.02 * rng.standard_normal((n, HID))).astype(np.float16).tobytes())
        if MASK_ID >= vocab:
            f.seek(MASK_ID * HID * 2)
            f.write((0.02 * rng.standard_normal(HID)).astype(np.float16).tobytes())
    lines.append(f"F embed.bin {rows_total * HID * 2}")

    with open(os.path.join(directory, "engine.idx"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return read_index(directory)


def check_layout(directory: str) -> list:
    """Every address `Engine::load` derives from the index (engine/engine.cu:166-275), checked against the files on
    disk. Returns the list of problems found (empty = loadable): a missing config key or tensor, a tensor or expert
    matrix that reaches past the end of its file, an offset that breaks the 16-byte alignment the loader's relayout and
    the GEMM's vector loads rely on, a vocabulary the readout kernels cannot slice, an embed.bin too short for the
    decoder's mask token."""
    bad = []
    ix = read_index(directory)
    need = ("num_hidden_layers", "vocab_size", "mask_id", "rms_norm_eps", "rope_theta", "routed_scaling_factor",
            "first_k_dense_replace", "nonexpert_bits", "lm_bits", "intermediate_size", "moe_intermediate_size")
    for k in need:
        if k not in ix.cfg:
            bad.append(f"config key {k} missing")
    if bad:
        return bad
    layers, vocab = int(ix.cfg["num_hidden_layers"]), int(ix.cfg["vocab_size"])
    first_moe, nb, lmb = int(ix.cfg["first_k_dense_replace"]), int(ix.cfg["nonexpert_bits"]), int(ix.cfg["lm_bits"])
    float(ix.cfg["rms_norm_eps"]), float(ix.cfg["rope_theta"]), float(ix.cfg["routed_scaling_factor"])

    def size(name):
        p = os.path.join(directory, name)
        if not os.path.exists(p):
            bad.append(f"file {name} missing")
            return 0
        n = os.path.getsize(p)
        if name in ix.fsize and ix.fsize[name] != n:
            bad.append(f"{name}: index says {ix.fsize[name]} bytes, file has {n}")
        return n

    def tensor(file, name, want_bytes, fbytes, align=16):
        try:
            t = ix.get(file, name)
        except KeyError as e:
            bad.append(str(e.args[0]))
            return
        if t.off % align:
            bad.append(f"{file}:{name} offset {t.off} not {align}-byte aligned")
        if t.off + want_bytes > fbytes:
            bad.append(f"{file}:{name} needs {want_bytes} bytes at {t.off}, file has {fbytes}")

    sb = size("small.bin")
    tensor("small.bin", "final_norm", HID * 4, sb, 4)
    tensor("small.bin", "signs", HID * 4, sb, 4)
    for li in range(layers):
        moe = li >= first_moe
        inter = int(ix.cfg["moe_intermediate_size" if moe else "intermediate_size"])
        if inter != (MOE_INTER if moe else INTER):
            bad.append(f"layer {li}: MLP width {inter}, the engine's buffers are sized for {MOE_INTER if moe else INTER}")
        for n, cnt in (("input_layernorm.weight", HID), ("post_attention_layernorm.weight", HID),
                       ("attention.query_layernorm.weight", HD), ("attention.key_layernorm.weight", HD)):
            tensor("small.bin", f"L{li}.{n}", cnt * 4, sb, 4)
        nef = f"nonexpert_L{li}.bin"
        neb = size(nef)
        for n, rows, k in (("qkv", QKV_ROWS, HID), ("dense", HID, HID), ("gate_up", 2 * inter, HID),
                           ("down", HID, inter)):
            tensor(nef, n, matrix_bytes(rows, k, nb), neb)
        if moe:
            tensor("small.bin", f"L{li}.router", NEXPERT * HID * 2, sb, 16)
            tensor("small.bin", f"L{li}.expert_bias", NEXPERT * 4, sb, 4)
            exb = size(f"experts_L{li}.bin")
            ex = ix.experts.get(li, [])
            if len(ex) != NEXPERT:
                bad.append(f"layer {li}: {len(ex)} expert lines, the engine indexes {NEXPERT}")
            for e, (bits, gu, dn) in enumerate(ex):
                if bits == 0:
                    continue
                if bits not in (2, 3, 4):
                    bad.append(f"layer {li} expert {e}: {bits} bits")
                    continue
                for what, off, nbytes in (("gate_up", gu, matrix_bytes(2 * inter, HID, bits)),
                                          ("down", dn, matrix_bytes(HID, inter, bits))):
                    if off % 16 or off < 0 or off + nbytes > exb:
                        bad.append(f"layer {li} expert {e} {what}: offset {off}, {nbytes} bytes, file has {exb}")
    if vocab % 128:
        bad.append(f"vocab_size {vocab} is not a multiple of 128")
    if lmb not in (2, 3, 4, 8) or nb not in (2, 3, 4, 8):
        bad.append(f"bit widths {nb} / {lmb}: the GEMM dispatches 2, 3, 4 and 8")
    else:
        tensor("lm_head.bin", "lm_head", matrix_bytes(vocab - vocab % 16, HID, lmb), size("lm_head.bin"))
    if size("embed.bin") < (max(vocab - 1, MASK_ID) + 1) * HID * 2:
        bad.append("embed.bin does not reach the mask token's row")
    return bad
