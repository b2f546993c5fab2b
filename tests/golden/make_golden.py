"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

Run in a container that has the reference checkout (it cannot travel to the GPU
box, the fixtures do):

    python tests/golden/make_golden.py /path/to/reference

Only ``ponyexl3.ref`` (numpy) is imported.  Everything written here comes out of
the reference's own functions; the seeds and shapes follow the reference's
tests (tests/test_codebook.py, tests/test_trellis.py,
tests/test_decode_reconstruct.py, tests/test_exl3_linear_module.py).
"""

from __future__ import annotations

import hashlib
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from ponyexl3.ref.codebook import CodebookMode, decode_3inst
    from ponyexl3.ref.decode import decode_packed_tile
    from ponyexl3.ref.forward import linear_forward_reconstruct
    from ponyexl3.ref.hadamard import had_r_128
    from ponyexl3.ref.perm import tensor_core_perm
    from ponyexl3.ref.reconstruct import reconstruct_inner
    from ponyexl3.ref.signs import unpack_sign_bitfield
    from ponyexl3.ref.synthetic import make_exl3_layer
    from ponyexl3.ref.trellis import (pack_trellis, pack_trellis_tile, unpack_trellis,
                                      unpack_trellis_tile)

    t0 = time.time()

    # ---- codebooks: every codeword of all three modes ------------------------------
    cbk: dict[str, np.ndarray] = {}
    for cb in CodebookMode:
        table = np.array([decode_3inst(w, cb) for w in range(65536)], dtype=np.float16)
        bits = table.view(np.uint16)
        cbk[f"sha256_{int(cb)}"] = np.frombuffer(
            hashlib.sha256(bits.tobytes()).digest(), dtype=np.uint8)
        cbk[f"stride16_{int(cb)}"] = bits[::16].copy()
        cbk[f"stats_{int(cb)}"] = np.array(
            [table.astype(np.float64).min(), table.astype(np.float64).max(),
             table.astype(np.float64).std()])
    cbk["probe_words"] = np.array([0, 1, 42, 0xABCD, 0xFFFF], dtype=np.uint32)
    cbk["probe_values"] = np.array(
        [[decode_3inst(int(w), cb) for w in cbk["probe_words"]] for cb in CodebookMode],
        dtype=np.float16).view(np.uint16)
    np.savez_compressed(HERE / "codebook.npz", **cbk)
    print(f"codebook tables done {time.time() - t0:.1f}s")

    # ---- trellis: literal per-tile unpack on arbitrary bitstreams + pack round trips --
    tr: dict[str, np.ndarray] = {"perm": tensor_core_perm()}
    for k in range(1, 9):
        rng = np.random.default_rng(4242 + k)
        packed = rng.integers(0, 65536, size=(4, 16 * k), dtype=np.uint16)
        packed[2] = 0xFFFF
        packed[3] = 0
        packed[3, 0] = 0x8001  # single marker bits to pin the bit order
        tr[f"packed_k{k}"] = packed
        tr[f"codewords_k{k}"] = np.stack([unpack_trellis_tile(p, k) for p in packed])
        # the reference's own round-trip inputs (tests/test_trellis.py:25-35)
        rng = np.random.default_rng(k)
        mask = (1 << k) - 1
        enc = (rng.integers(0, 2**16, size=256, dtype=np.uint32) & mask).astype(np.uint16)
        tr[f"encoded_k{k}"] = enc
        tr[f"encoded_packed_k{k}"] = pack_trellis_tile(enc, k)
        # tensor form (tests/test_trellis.py:50-57)
        rng = np.random.default_rng(99 + k)
        enc3 = (rng.integers(0, 2**16, size=(2, 3, 256), dtype=np.uint32) & mask).astype(np.uint16)
        p3 = pack_trellis(enc3, k)
        tr[f"encoded3_k{k}"] = enc3
        tr[f"packed3_k{k}"] = p3
        tr[f"codewords3_k{k}"] = unpack_trellis(p3, k)
    np.savez_compressed(HERE / "trellis.npz", **tr)

    # ---- decoded tiles: one arbitrary tile per (K, codebook) --------------------------
    tl: dict[str, np.ndarray] = {}
    for k in range(1, 9):
        for cb in CodebookMode:
            rng = np.random.default_rng(100 * k + int(cb))
            packed = rng.integers(0, 65536, size=16 * k, dtype=np.uint16)
            tl[f"packed_k{k}_cb{int(cb)}"] = packed
            tl[f"tile_k{k}_cb{int(cb)}"] = decode_packed_tile(packed, k, cb).view(np.uint16)
    np.savez_compressed(HERE / "tiles.npz", **tl)
    print(f"trellis + tiles done {time.time() - t0:.1f}s")

    # ---- Hadamard -----------------------------------------------------------------
    rng = np.random.default_rng(77)
    hx = rng.standard_normal((3, 384)).astype(np.float16)
    pre = np.where(rng.random(384) > 0.5, -1.0, 1.0).astype(np.float16)
    post = (rng.standard_normal(384) * 0.5).astype(np.float16)
    hd = {
        "x": hx.view(np.uint16), "pre": pre.view(np.uint16), "post": post.view(np.uint16),
        "y_plain": had_r_128(hx.astype(np.float32)),
        "y_pre": had_r_128(hx.astype(np.float32), pre_scale=pre),
        "y_post": had_r_128(hx.astype(np.float32), post_scale=post),
        "y_both": had_r_128(hx.astype(np.float32), pre_scale=pre, post_scale=post),
        "sign_words": np.array([0x0001, 0x8000, 0xA5A5, 0x0000, 0xFFFF, 0x1234], dtype=np.uint16),
    }
    hd["sign_values"] = unpack_sign_bitfield(hd["sign_words"].view(np.int16)).view(np.uint16)
    np.savez_compressed(HERE / "hadamard.npz", **hd)

    # ---- whole forwards through linear_forward_reconstruct ----------------------------
    fw: dict[str, np.ndarray] = {}
    cases = []
    for k in range(1, 9):
        for cbi, (mcg, mul1) in enumerate([(False, False), (True, False), (False, True)]):
            cases.append(dict(k=k, mcg=mcg, mul1=mul1, inf=128, outf=128, rows=2, bias=False,
                              seed=10 * k + cbi, xs=1.0))
    # shapes of the reference's module test (tests/test_exl3_linear_module.py:21-35)
    cases.append(dict(k=4, mcg=True, mul1=False, inf=256, outf=384, rows=4, bias=True, seed=15, xs=0.5))
    cases.append(dict(k=2, mcg=True, mul1=False, inf=256, outf=384, rows=16, bias=True, seed=13, xs=0.5))
    cases.append(dict(k=5, mcg=False, mul1=False, inf=384, outf=256, rows=1, bias=True, seed=21, xs=1.0))
    cases.append(dict(k=4, mcg=True, mul1=True, inf=128, outf=256, rows=3, bias=False, seed=22, xs=1.0))
    names = []
    for i, c in enumerate(cases):
        layer = make_exl3_layer(k=c["k"], in_features=c["inf"], out_features=c["outf"],
                                seed=c["seed"], mcg=c["mcg"], mul1=c["mul1"], bias=c["bias"])
        rng = np.random.default_rng(1000 + i)
        x = (rng.standard_normal((c["rows"], c["inf"])) * c["xs"]).astype(np.float16)
        y = linear_forward_reconstruct(layer, x)
        w = reconstruct_inner(layer.trellis, layer.k, mcg=layer.mcg, mul1=layer.mul1)
        n = f"c{i}"
        names.append(n)
        fw[f"{n}_meta"] = np.array([c["k"], int(c["mcg"]), int(c["mul1"]), c["inf"], c["outf"],
                                    c["rows"], int(c["bias"])], dtype=np.int64)
        fw[f"{n}_trellis"] = layer.trellis
        fw[f"{n}_suh"] = layer.suh.view(np.uint16)
        fw[f"{n}_svh"] = layer.svh.view(np.uint16)
        if layer.bias is not None:
            fw[f"{n}_bias"] = layer.bias.astype(np.float16).view(np.uint16)
        fw[f"{n}_x"] = x.view(np.uint16)
        fw[f"{n}_y"] = y.view(np.uint16)
        fw[f"{n}_w_sha256"] = np.frombuffer(
            hashlib.sha256(np.ascontiguousarray(w).view(np.uint16).tobytes()).digest(),
            dtype=np.uint8)
        print(f"forward case {i} {c} done {time.time() - t0:.1f}s")
    # one case with the legacy packed int16 sign words (ponyexl3/ref/signs.py:8-19)
    layer = make_exl3_layer(k=3, in_features=128, out_features=128, seed=31)
    rng = np.random.default_rng(31)
    su = rng.integers(0, 65536, size=128 // 16, dtype=np.uint16).view(np.int16)
    sv = rng.integers(0, 65536, size=128 // 16, dtype=np.uint16).view(np.int16)
    layer.suh, layer.svh = su, sv
    x = rng.standard_normal((2, 128)).astype(np.float16)
    fw["packed_signs_trellis"] = layer.trellis
    fw["packed_signs_su"] = su
    fw["packed_signs_sv"] = sv
    fw["packed_signs_x"] = x.view(np.uint16)
    fw["packed_signs_y"] = linear_forward_reconstruct(layer, x).view(np.uint16)
    fw["n_cases"] = np.array([len(names)])
    np.savez_compressed(HERE / "forward.npz", **fw)
    encoder(ref_root)
    print(f"all done {time.time() - t0:.1f}s")


def encoder(ref_root: str) -> None:
    """Trellis search of single tiles by the reference's exact Viterbi
    (ponyexl3/convert/reference_search.py); seeds and K follow tests/test_convert.py, plus more
    K, the other two codebooks and tiles whose first free pass does not close."""
    sys.path.insert(0, ref_root)
    from ponyexl3.convert.reference_search import quantize_tile_reference
    from ponyexl3.ref.codebook import CodebookMode

    t0 = time.time()
    modes = {0: CodebookMode.DEFAULT, 1: CodebookMode.MCG, 2: CodebookMode.MUL1}
    cases = [(2, 0, 7, 1.0), (3, 0, 7, 1.0), (4, 0, 11, 1.0), (3, 1, 12, 1.0), (4, 2, 13, 1.0), (1, 0, 14, 1.0),
             (2, 0, 15, 3.0), (5, 0, 16, 0.7)]
    enc = {"n_cases": np.array([len(cases)])}
    for i, (k, cb, seed, scale) in enumerate(cases):
        w = (np.random.default_rng(seed).standard_normal(256) * scale).astype(np.float32)
        states, decoded = quantize_tile_reference(w, k=k, cb=modes[cb])
        enc[f"c{i}_k"], enc[f"c{i}_cb"] = np.array([k]), np.array([cb])
        enc[f"c{i}_w"], enc[f"c{i}_states"], enc[f"c{i}_decoded"] = w, states.astype(np.uint16), decoded
        print(f"encoder case {i}: k={k} cb={cb} mse={float(((decoded - w) ** 2).mean()):.5f} {time.time() - t0:.1f}s")
    np.savez_compressed(HERE / "encoder.npz", **enc)


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[2] == "encoder":      # only the (slow) trellis-search cases
        encoder(sys.argv[1])
    elif len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of the reference project> [encoder]")
    else:
        main(sys.argv[1])
