"""Generates tests/golden/*.npz by running the REFERENCE's own NumPy functions.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference [--config1]

It loads ``nectarml/cpu/conv/conv2d.py`` from that checkout on its own (the six ``_conv*``
functions only need NumPy; ``nectarml.typing.float32`` is stubbed) and ``nectarml/cpu/math.py``
for ``matmul``.  Linear gradients follow nectarml/core/_tensor/numerical.py:896-904 with
``cpu.math.matmul`` as the product, because the reference's CPU autograd for matmul raises
(nectarml/core/_tensor/fake.py:94-97).  ``--config1`` adds the full-size benchmark configuration 1
forward, which takes several minutes in the reference's pure-Python loop.
"""
import importlib.util
import os
import sys
import time
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def load_reference(root):
    pkg = types.ModuleType("nectarml")
    pkg.__path__ = []
    typing_stub = types.ModuleType("nectarml.typing")
    typing_stub.float32 = "float32"
    sys.modules.setdefault("nectarml", pkg)
    sys.modules.setdefault("nectarml.typing", typing_stub)
    mods = {}
    for name, rel in (("conv2d", "nectarml/cpu/conv/conv2d.py"), ("math", "nectarml/cpu/math.py")):
        spec = importlib.util.spec_from_file_location("_ref_" + name, os.path.join(root, rel))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        mods[name] = m
    return mods["conv2d"], mods["math"]


class _T:  # the minimal Tensor the reference's cpu.math functions read: a .data attribute
    def __init__(self, a):
        self.data = a


def run_conv_case(ref, name, case, want_forward=True):
    transposed, geom, has_bias, _ = case
    B, Ci, H, W, Co, KH, KW, s, p, d, op = geom
    x, w, b, dy = cases.draw_conv(name, case) if name != "config1" else cases.draw_conv(name, case, cases.CONFIG1_SEED)
    Ho, Wo = cases.out_hw(transposed, geom)
    out = {}
    if not transposed:
        if want_forward:
            y, x_pad = ref._conv2d(x, w, b, B, Ci, H, W, Co, KH, KW, Ho, Wo, s[0], s[1], p[0], p[1], d[0], d[1], 1)
            out["y"] = y
        else:
            x_pad = np.pad(x, ((0, 0), (0, 0), (p[0], p[0]), (p[1], p[1]))) if (p[0] or p[1]) else x
        out["dx"] = ref._conv2d_backward_input(dy, x_pad, w, KH, KW, Ho, Wo, s[0], s[1], p[0], p[1], d[0], d[1], 1)
        out["dw"] = ref._conv2d_backward_weight(dy, x_pad, w, KH, KW, Ho, Wo, s[0], s[1], d[0], d[1], 1)
    else:
        out["y"] = ref._conv_transpose2d(x, w, b, B, Ci, H, W, Co, KH, KW, s[0], s[1], p[0], p[1], d[0], d[1],
                                         op[0], op[1], 1)
        out["dx"] = ref._conv_transpose2d_backward_input(dy, w, B, Ci, H, W, Co, KH, KW, Ho, Wo, s[0], s[1], p[0],
                                                         p[1], d[0], d[1], 1)
        out["dw"] = ref._conv_transpose2d_backward_weight(dy, x, B, Ci, H, W, Co, KH, KW, Ho, Wo, s[0], s[1], p[0],
                                                          p[1], d[0], d[1], 1)
    out["db"] = dy.sum(axis=(0, 2, 3))  # nectarml/cpu/conv/conv2d.py:64-67
    return (x, w, b, dy), out


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not args:
        raise SystemExit("usage: make_golden.py <path of the reference checkout> [--config1]")
    root = args[0]
    ref, ref_math = load_reference(root)
    if "--conv1d" in sys.argv:
        # the reference's 1-D functions (nectarml/cpu/conv/conv1d.py:20-215), its own file
        spec = importlib.util.spec_from_file_location("_ref_conv1d", os.path.join(root, "nectarml/cpu/conv/conv1d.py"))
        r1 = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(r1)
        s1 = {}
        for name, case in cases.CONV1D_CASES.items():
            transposed, (B, Ci, L, Co, K, st, p, d, op), _ = case
            x, w, b, dy = cases.draw_conv1d(name, case)
            Lo = dy.shape[2]
            if not transposed:
                y, x_pad = r1.conv1d(x, w, b, B, Ci, Lo, Co, K, st, p, d, 1)
                dx = r1.conv1d_backward_input(dy, x_pad, w, st, p, d, 1)
                dw = r1.conv1d_backward_weight(dy, x_pad, w, st, p, d, 1)
            else:
                y = r1.conv_transpose1d(x, w, b, B, Ci, L, Co, K, st, p, d, op, 1)
                dx = r1.conv_transpose1d_backward_input(dy, w, B, Ci, L, Co, K, Lo, st, p, d, 1)
                dw = r1.conv_transpose1d_backward_weight(dy, x, B, Ci, L, Co, K, Lo, st, p, d, 1)
            for k, v in (("y", y), ("dx", dx), ("dw", dw), ("db", dy.sum(axis=(0, 2)))):
                s1[f"{name}__{k}"] = np.asarray(v, np.float32)
            s1[f"{name}__insum"] = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
            print(name, y.shape, dx.shape, dw.shape)
        np.savez_compressed(os.path.join(HERE, "conv1d_cases.npz"), **s1)
        return
    store = {}
    for name, case in cases.CONV_CASES.items():
        (x, w, b, dy), out = run_conv_case(ref, name, case)
        for k, v in out.items():
            store[f"{name}__{k}"] = np.asarray(v, np.float32)
        store[f"{name}__insum"] = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
        print(name, {k: v.shape for k, v in out.items()})
    for name, shape in cases.LINEAR_CASES.items():
        x, w, b, dy = cases.draw_linear(name, shape)
        y = b + ref_math.matmul(_T(x), _T(np.ascontiguousarray(w.T)))          # nn/linear.py:44-47
        dx = ref_math.matmul(_T(dy), _T(w))                                    # numerical.py:896-899
        dw = ref_math.matmul(_T(np.ascontiguousarray(dy.T)), _T(x))            # numerical.py:900-904 (as dW of W)
        store[f"{name}__y"], store[f"{name}__dx"], store[f"{name}__dw"] = y, dx, dw
        store[f"{name}__db"] = dy.sum(axis=0)
        store[f"{name}__insum"] = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
    np.savez_compressed(os.path.join(HERE, "small_cases.npz"), **store)
    print("wrote small_cases.npz", sum(v.nbytes for v in store.values()), "bytes raw")

    if "--config1" in sys.argv:
        t0 = time.time()
        (x, w, b, dy), out = run_conv_case(ref, "config1", cases.CONFIG1)
        print("config1 reference run: %.1f s" % (time.time() - t0))
        s1 = {}
        for k in ("y", "dx", "dw"):
            flat = np.asarray(out[k], np.float32).reshape(-1)
            idx = cases.sample_indices(flat.size, cases.CONFIG1_SAMPLES, 11 + len(k))
            s1[f"{k}_idx"], s1[f"{k}_val"] = idx, flat[idx]
            s1[f"{k}_sum"] = np.array([flat.sum(dtype=np.float64), np.abs(flat).sum(dtype=np.float64)])
        s1["db"] = np.asarray(out["db"], np.float32)
        s1["insum"] = np.array([x.sum(dtype=np.float64), w.sum(dtype=np.float64), dy.sum(dtype=np.float64)])
        s1["reference_seconds"] = np.array([time.time() - t0])
        np.savez_compressed(os.path.join(HERE, "config1_samples.npz"), **s1)
        print("wrote config1_samples.npz")


if __name__ == "__main__":
    main()
