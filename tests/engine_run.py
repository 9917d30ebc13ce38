"""Child process of test_gpu_engine_dir.py: start one build of the reference engine library on a synthetic engine
directory and generate from a seeded prompt, the way the reference's server binds and calls it
(`server/server.py:62-71,94-117`: `llada_init`, `llada_generate`, `llada_stats` over ctypes). Prints one JSON line.
The engine ends the process on a malformed directory (`exit(1)` in its loader), which is why it runs in a child.

    python tests/engine_run.py <libllada*.so> <engine directory> <prompt tokens> <new tokens> [<vocab> [<max context tokens>]]
"""
import ctypes
import json
import sys
import time

import numpy as np


def main():
    lib_path, directory, nprompt, max_new = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
    vocab = int(sys.argv[5]) if len(sys.argv) > 5 else 4096
    max_ctx = int(sys.argv[6]) if len(sys.argv) > 6 else 4096
    lib = ctypes.CDLL(lib_path)
    cb_t = ctypes.CFUNCTYPE(None, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_void_p)
    lib.llada_init.restype = ctypes.c_void_p
    lib.llada_init.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.llada_generate.restype = ctypes.c_int
    lib.llada_generate.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int,
                                   ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                   ctypes.POINTER(ctypes.c_int), ctypes.c_int, cb_t, ctypes.c_void_p]
    lib.llada_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_double)]
    t0 = time.time()
    h = lib.llada_init(directory.encode(), max_ctx)
    load_s = time.time() - t0
    prompt = np.random.default_rng(7).integers(0, vocab, nprompt).astype(np.int32)
    blocks = []

    def on_block(ptr, n, _user):
        blocks.append([ptr[i] for i in range(n)])

    runs = []
    for _ in range(2):                                   # the second call meets the first one's committed prefix
        arr = (ctypes.c_int * nprompt)(*prompt.tolist())
        out = (ctypes.c_int * (max_new + 64))()
        t0 = time.time()
        n = lib.llada_generate(h, arr, nprompt, max_new, 0.5, 0.0, 16, 32, out, len(out), cb_t(on_block), None)
        s = (ctypes.c_double * 8)()
        lib.llada_stats(h, s)
        runs.append({"ids": list(out[:n]), "seconds": time.time() - t0, "steps": s[0], "blocks": s[1],
                     "commits": s[2], "reused_blocks": s[3], "weights_gb": s[4], "kv_gb": s[5], "max_ctx": s[6]})
    print(json.dumps({"load_s": load_s, "runs": runs, "streamed": sum(len(b) for b in blocks)}))


if __name__ == "__main__":
    main()
