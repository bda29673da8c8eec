"""Record the reference's accept / reject decision for every call in ``gate_cases.cases()``.

Run where a checkout of the reference is at hand:
    python tests/golden/gen_supported_golden.py <path to the reference checkout>
It imports the reference's own ``kuipy`` package (pure Python; no kernel is built or run),
hands its ``supported()`` gates fake-CUDA tensors and writes ``supported_golden.json`` next to
this file: one entry per case with ``accept`` (true / false).  Also records the reference's
tile choosers on the mm shapes and its ``_verify_compare`` metric on seeded tensors
(``verify_golden.json``).
"""
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

from fake_cuda import FakeCudaTensor  # noqa: E402
from gate_cases import DT, cases  # noqa: E402


def materialise(d):
    if isinstance(d, tuple) and d and d[0] == "T":
        return FakeCudaTensor(torch.zeros(d[1], dtype=DT[d[2]]))
    if isinstance(d, tuple) and d and d[0] == "CPU":
        return torch.zeros(d[1], dtype=DT[d[2]])
    if isinstance(d, tuple) and d and d[0] == "L":
        return [materialise(x) for x in d[1]]
    return d


def resolve(op_name):
    packet, overload = op_name.split(".")
    return getattr(getattr(torch.ops.aten, packet), overload)


def main(ref_root):
    sys.path.insert(0, ref_root)
    import kuipy                      # the reference package
    from kuipy import kuiops as ref
    assert Path(kuipy.__file__).resolve().is_relative_to(Path(ref_root).resolve()), kuipy.__file__
    fams = {}
    rows = []
    for fam, op, args, kwargs in cases():
        impl = fams.setdefault(fam, getattr(ref, fam)({}))
        spec = impl.supported(resolve(op), tuple(materialise(a) for a in args), dict(kwargs))
        rows.append({"family": fam, "op": op, "accept": spec is not None})
    tiles = []
    for dt in ("f32", "bf16", "f16"):
        for M, N, K in [(64, 64, 64), (128, 64, 128), (128, 63, 128), (32, 32, 32), (16, 4096, 4096), (4096, 4096, 4096),
                        (96, 64, 64), (64, 64, 16), (64, 64, 8), (256, 128, 32), (192, 192, 192)]:
            tiles.append({"dtype": dt, "M": M, "N": N, "K": K,
                          "bt2d": ref._bt2d_tile(DT[dt], M, N, K), "tc2d": ref._tc2d_tile(DT[dt], M, N, K)})
    (HERE / "supported_golden.json").write_text(json.dumps({"cases": rows, "tiles": tiles}, indent=0))

    # verify-mode metric on seeded tensors
    class F:
        def __init__(self, n): self.n = n
        def __str__(self): return self.n
    g = torch.Generator().manual_seed(0)
    recs = []
    for i, noise in enumerate([0.0, 1e-3, 1e-2, 5e-2, 0.5]):
        a = torch.randn(16, 24, generator=g)
        b = a + noise * torch.randn(16, 24, generator=g)
        kuipy.reset_verify()
        kuipy._verify_compare(F(f"op{i}"), a, b, 2e-2)
        st = kuipy.verify_stats[f"op{i}"]
        recs.append({"noise": noise, "n": st["n"], "fail": st["fail"], "max_rel": st["max_rel"]})
    (HERE / "verify_golden.json").write_text(json.dumps({"seed": 0, "shape": [16, 24], "tol": 2e-2, "records": recs}, indent=0))
    print(f"{len(rows)} gate cases, {sum(r['accept'] for r in rows)} accepted; {len(tiles)} tile records")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
