"""Generate the golden fixtures in this folder by running the REFERENCE's own Python code.

Run once, in a container that has the reference checkout (its root in ``ACTNN_REFERENCE_ROOT``):

    python oracle/build_ref.py            # the reference's calc_precision.cc, unmodified
    python tests/golden/make_golden.py

What runs is the reference's ``actnn/actnn/ops.py`` (simulate branch of
``quantize_and_pack`` / ``dequantize_and_unpack``, ``quantize_activation`` /
``dequantize_activation``), ``qscheme.py`` and ``qbnscheme.py``, loaded from the checkout
without executing ``actnn/__init__.py`` (which needs ``torch._six`` and the CUDA build).
The compiled extensions those files import are replaced as follows:

* ``actnn.cpp_extension.calc_precision`` -> the reference's own C++ built by
  ``oracle/build_ref.py``;
* ``actnn.cpp_extension.minimax`` -> ``torch.min/max(dim=1)``, the meaning the reference's
  ``tests/test_minimax.py:19-30`` pins for that kernel;
* ``actnn.cpp_extension.quantization`` / ``backward_func`` -> empty stand-ins (never called
  on the simulate branch);
* ``Tensor.cuda()`` -> identity, and ``torch.ones(..., device='cuda')`` (``ops.py:28``)
  -> the same call on the CPU, so the scheme and glue code run on CPU tensors.

The reference draws its rounding noise with ``uniform_(-0.5, 0.5)`` from the default
generator; this script reseeds that generator right before each call and records the
noise a same-seeded draw of the same shape and dtype yields, so the fixtures carry the
exact noise the reference used.

Output: ``tests/golden/*.npz`` (small cases only; bfloat16 / float16 tensors are stored as
their raw uint16 bit patterns).
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = os.environ.get("ACTNN_REFERENCE_ROOT")
if not REFERENCE:
    raise SystemExit("set ACTNN_REFERENCE_ROOT to the root of a checkout of the reference")
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def load_reference():
    import build_ref

    ref_cp = build_ref.load_ref_calc_precision()
    if ref_cp is None:
        raise SystemExit("run `python oracle/build_ref.py` first")

    pkg_dir = os.path.join(REFERENCE, "actnn", "actnn")
    pkg = types.ModuleType("actnn")
    pkg.__path__ = [pkg_dir]
    sys.modules["actnn"] = pkg
    ext = types.ModuleType("actnn.cpp_extension")
    ext.__path__ = []
    sys.modules["actnn.cpp_extension"] = ext

    mm = types.ModuleType("actnn.cpp_extension.minimax")
    mm.minimax = lambda data: (torch.min(data, 1)[0], torch.max(data, 1)[0])
    sys.modules["actnn.cpp_extension.minimax"] = mm
    sys.modules["actnn.cpp_extension.calc_precision"] = ref_cp
    for name in ("quantization", "backward_func"):
        sys.modules["actnn.cpp_extension." + name] = types.ModuleType("actnn.cpp_extension." + name)
    ext.minimax, ext.calc_precision = mm, ref_cp

    torch.Tensor.cuda = lambda self, *a, **k: self      # CPU stand-in for .cuda()
    real_ones = torch.ones

    def ones_on_cpu(*a, **k):
        if k.get("device") == "cuda":
            k.pop("device")
        return real_ones(*a, **k)
    torch.ones = ones_on_cpu

    import actnn.conf as conf
    import actnn.ops as ops
    import actnn.qscheme as qscheme
    import actnn.qbnscheme as qbnscheme
    pkg.QBNScheme = qbnscheme.QBNScheme
    conf.config.simulate = True
    return conf.config, ops, qscheme.QScheme, qbnscheme.QBNScheme


def raw(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def main():
    config, ops, QScheme, QBNScheme = load_reference()
    out = {}

    # ---- 1. quantize_and_pack / dequantize_and_unpack, simulate branch (ops.py:22-74) ----
    case = 0
    for dname, dt in DT.items():
        for kind in ("relu", "randn", "wide"):
            for bits_kind in ("mixed", 1, 2, 4, 8):
                n, g, gs = 5, 3, 256
                torch.manual_seed(100 + case)
                x = torch.randn(n, g, gs)
                if kind == "relu":
                    x = torch.relu(x)
                elif kind == "wide":
                    x = x * torch.tensor([0.05, 1.0, 30.0, 1e3, 7.0]).view(n, 1, 1) + 3.0
                x = x.to(dt)
                mn, mx = torch.min(x, 2, keepdim=True)[0], torch.max(x, 2, keepdim=True)[0]
                if bits_kind == "mixed":
                    bits = torch.tensor([1, 2, 3, 8, 5], dtype=torch.int32)
                else:
                    bits = torch.ones(n, dtype=torch.int32) * bits_kind
                seed = 1000 + case
                torch.manual_seed(seed)
                noise = torch.empty(x.shape, dtype=dt).uniform_(-0.5, 0.5)
                torch.manual_seed(seed)
                codes, scale = ops.quantize_and_pack(x, bits, mn, mx)
                deq = ops.dequantize_and_unpack(codes, x.shape, bits, scale, mn)
                key = f"q_{dname}_{kind}_{bits_kind}"
                for nm, t in (("x", x), ("mn", mn), ("mx", mx), ("noise", noise), ("scale", scale), ("deq", deq)):
                    out[f"{key}__{nm}"] = raw(t)
                out[f"{key}__bits"] = bits.numpy()
                out[f"{key}__codes"] = codes.numpy().astype(np.uint8)
                assert codes.max() <= 255 and codes.min() >= 0
                case += 1
    np.savez_compressed(os.path.join(HERE, "quantize_simulate.npz"), **out)
    print("quantize_simulate:", case, "cases")

    # ---- 2. quantize_activation / dequantize_activation through the schemes ----
    out = {}
    config.perlayer = False
    case = 0
    for dname, dt in DT.items():
        for which in ("conv", "bn", "none"):
            for shape in ((6, 8, 7, 9), (4, 16, 8, 8), (3, 10)):
                torch.manual_seed(200 + case)
                x = (torch.randn(*shape) * torch.exp(torch.randn(shape[0]).view(-1, *([1] * (len(shape) - 1))))).to(dt)
                if which == "conv":
                    config.activation_compression_bits = [2, 8, 8]
                    scheme = QScheme(None, num_locations=9)
                    scheme.scales = torch.tensor(0.37)      # as left by set_scale (qscheme.py:55)
                elif which == "bn":
                    config.activation_compression_bits = [2, 8, 8]
                    scheme = QBNScheme()
                else:
                    config.activation_compression_bits = [4]
                    scheme = None
                seed = 2000 + case
                n = shape[0]
                f = int(np.prod(shape[1:]))
                fpad = (f + 255) // 256 * 256
                torch.manual_seed(seed)
                noise = torch.empty((n, fpad // 256, 256), dtype=dt).uniform_(-0.5, 0.5)
                torch.manual_seed(seed)
                q = ops.quantize_activation(x, scheme)
                deq = ops.dequantize_activation(q, x.shape)
                codes, q_bits, q_scale, q_min = q
                key = f"a_{dname}_{which}_{'x'.join(map(str, shape))}"
                out[f"{key}__x"] = raw(x)
                out[f"{key}__noise"] = raw(noise)
                out[f"{key}__codes"] = codes.numpy().astype(np.uint8)
                out[f"{key}__bits"] = (np.array([q_bits] * n, dtype=np.int32) if isinstance(q_bits, int)
                                        else q_bits.numpy().astype(np.int32))
                out[f"{key}__scale"] = raw(q_scale)
                out[f"{key}__min"] = raw(q_min)
                out[f"{key}__deq"] = raw(deq)
                if which == "conv":
                    out[f"{key}__C"] = scheme.C.numpy()
                case += 1
    np.savez_compressed(os.path.join(HERE, "quantize_activation.npz"), **out)
    print("quantize_activation:", case, "cases")

    # ---- 3. calc_precision.cc (the reference's compiled greedy) ----
    out = {}
    cp = sys.modules["actnn.cpp_extension.calc_precision"]
    torch.manual_seed(7)
    for t in range(40):
        n = [1, 2, 7, 64, 256, 512][t % 6]
        kind = t % 5
        if kind == 0:
            C = torch.zeros(n)
        elif kind == 1:
            C = torch.exp(torch.randn(n))                  # LogNormal(0, 1)
        elif kind == 2:
            C = torch.exp(torch.randn(n)) * 1e-42          # denormal priorities
        elif kind == 3:
            C = torch.randint(0, 3, (n,)).float()          # heavy ties
        else:
            C = torch.exp(torch.randn(n) * 5)
        weighted = t % 8 == 7
        w = torch.randint(1, 5000, (n,), dtype=torch.int32) if weighted else torch.ones(n, dtype=torch.int32)
        avg = [2.0, 1.0, 8.0, 3.3, 1.5, 9.0, 2.0, 4.0][t % 8]
        target = int(avg * int(w.sum()))
        b = cp.calc_precision(torch.ones(n, dtype=torch.int32) * 8, C.clone(), w.clone(), target)
        out[f"g{t}__C"] = C.numpy()
        out[f"g{t}__w"] = w.numpy()
        out[f"g{t}__target"] = np.array([target], dtype=np.int64)
        out[f"g{t}__b"] = b.numpy().astype(np.int8)
    np.savez_compressed(os.path.join(HERE, "calc_precision.npz"), **out)
    print("calc_precision: 40 cases")

    # ---- 4. per-layer re-allocation (qscheme.py:96-128, qbnscheme.py:54-60) ----
    # Both branches of QScheme.allocate_perlayer: the joint allocation over layers x samples
    # (group bits != initial bits: each layer gets the mean width of its samples) and the
    # one-width-per-layer allocation (group bits == initial bits), then the batch-norm schemes
    # that copy the width of the conv / linear layer in front of them.
    out = {}
    config.perlayer = True
    case = 0
    for group_bits, initial_bits, L, N in ((2, 8, 4, 6), (2, 8, 7, 16), (3, 8, 5, 8), (4, 4, 5, 6), (8, 8, 3, 4),
                                           (2, 2, 4, 5)):
        QScheme.layers.clear()
        QBNScheme.layers.clear()
        config.activation_compression_bits = [group_bits]
        config.initial_bits = initial_bits
        torch.manual_seed(400 + case)
        dims = torch.randint(1, 40, (L,)) * 256
        Cs = torch.exp(torch.randn(L, N) * 1.5) * torch.exp(torch.randn(L, 1))
        follows = []
        for i in range(L):
            layer = QScheme(None)
            layer.C = Cs[i].clone()
            layer.dim = int(dims[i])
            if i % 2 == 0:
                bn = QBNScheme()                               # prev_linear = the layer just made
                follows.append(i)
        QScheme.allocate_perlayer()
        QBNScheme.allocate_perlayer()
        key = f"p{case}"
        out[f"{key}__C"] = Cs.numpy()
        out[f"{key}__dims"] = dims.numpy().astype(np.int64)
        out[f"{key}__cfg"] = np.array([group_bits, initial_bits], dtype=np.int64)
        out[f"{key}__bits"] = np.array([float(layer.bits) for layer in QScheme.layers], dtype=np.float32)
        out[f"{key}__bn_follows"] = np.array(follows, dtype=np.int64)
        out[f"{key}__bn_bits"] = np.array([float(bn.bits) for bn in QBNScheme.layers], dtype=np.float32)
        case += 1
    QScheme.layers.clear()
    QBNScheme.layers.clear()
    np.savez_compressed(os.path.join(HERE, "perlayer.npz"), **out)
    print("perlayer:", case, "cases")


if __name__ == "__main__":
    main()
