"""One forward at a benchmark geometry through this library and through the reference's production CUDA
build (oracle/_ref/libo1ref.so, cuBLASLt + cuDNN SDPA) on the same seeded weights and inputs; prints one
JSON line with the distance of x_pred and of the block checkpoints.  bench.py runs it as a child process
after its timed region, so the benchmark process itself never maps the reference build.

  python tests/parity_probe.py [--text 256 --grid-h 128 --grid-w 128 --layers 2 --weights A]
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--text", type=int, default=256)
    ap.add_argument("--grid-h", type=int, default=128)
    ap.add_argument("--grid-w", type=int, default=128)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--weights", default="A", choices=["A", "B"])
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    out = {"against": "reference CUDA build (cuBLASLt + cuDNN SDPA), same seeded weights and inputs",
           "rows": a.text + a.grid_h * a.grid_w, "layers": a.layers, "weights": a.weights}
    try:
        import torch
        import parity
        if parity.reflib() is None:
            out["status"] = "reference build absent"
            print(json.dumps(out))
            return 0
        import refharness as rh
        from __graft_entry__ import load_package
        pkg = load_package()
        torch.cuda.set_device(a.device)
        dev = torch.device("cuda", a.device)
        pkg.use_torch_stream()
        T, gh, gw = a.text, a.grid_h, a.grid_w
        I = gh * gw
        w = pkg.Weights(n_layers=a.layers, seed=1234, weight_set=a.weights, device=dev)
        eng = pkg.Engine(w, T, I)
        reng = rh.RefEngine(w.binding, T, gh, gw, dev, production=True)
        ids = rh.seeded_ids(T)[0].to(dev)
        z = rh.seeded_latent(I).to(dev)
        pos, _ = pkg.seq_t2i(T, gh, gw)
        names = ("after_block_0", "after_final_norm")
        mine, md = eng.forward(ids, pos.to(dev), z, 0.5, diag_names=names)
        theirs = torch.empty_like(mine)
        rd = reng.forward(ids, z, 0.5, theirs, diag_names=names)
        torch.cuda.synchronize()
        assert pkg.lib.o1_device_error() == 0
        reng.close()
        for key, g, r in (("after_block_0", md["after_block_0"], rd["after_block_0"]),
                          ("after_final_norm", md["after_final_norm"], rd["after_final_norm"]),
                          ("x_pred", mine, theirs), ("x_pred_image_rows", mine[T:], theirs[T:])):
            n, c, m, bad = parity.metrics_dev(g, r)
            out[key] = {"nrmse": round(n, 6), "cos": round(c, 7), "max_abs": round(m, 5), "nonfinite": bad}
        b0, xp = out["after_block_0"], out["x_pred"]
        # per-block bar of the path: NRMSE <= 1e-2, cosine >= 0.999; whole-model output envelope of
        # o1.c tests/unit/test_full_forward.c:484: NRMSE <= 0.18, cosine >= 0.99
        ok = (b0["nrmse"] <= 1e-2 and b0["cos"] >= 0.999 and xp["nrmse"] <= 0.18 and xp["cos"] >= 0.99 and
              not b0["nonfinite"] and not xp["nonfinite"])
        out["status"] = "pass" if ok else "FAIL"
    except Exception as ex:          # noqa: BLE001 -- the probe reports, the bench line carries the text
        out["status"] = f"error: {type(ex).__name__}: {ex}"
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
