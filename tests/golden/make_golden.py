"""Generate the committed golden vectors from the reference's own CPU operators.

Needs `oracle/_ref/_apr_ref*.so` (python oracle/build_ref.py), i.e. the reference checkout.  For a few
small seeded structures it stores the access arrays, seeded inputs and the outputs of every operator
as computed by the reference code in float64, one .npz per structure.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (os.path.join(ROOT, "apr-cnn_b200", "pyapr"), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, p)

import synthetic  # noqa: E402  (imported stand-alone: no GPU extension needed)
import ref  # noqa: E402

CASES = {"odd": ((13, 9, 21), 3, 0.05), "cube16": ((16, 16, 16), 1, 0.03), "plane": ((1, 33, 31), 5, 0.1),
         "odd2": ((20, 11, 12), 9, 0.2)}
CIN, COUT, NST = 3, 4, 2


def main():
    m = ref.load()
    assert m is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    for name, (shape, seed, dens) in CASES.items():
        a = synthetic.random_apr(shape, seed, density=dens)
        apr = ref.make_apr(m, a)
        L = a.level_max - a.level_min + 1
        out = dict(shape=np.array(shape), level_min=a.level_min, level_max=a.level_max, dims=np.array(a.dims),
                   row_ptr=a.row_ptr, y=a.y, tree_row_ptr=a.tree_row_ptr, tree_y=a.tree_y)
        rng = np.random.RandomState(1000 + seed)
        dls = []
        for dl in range(0, 3):
            cml = a.level_max - dl
            if cml - 1 < a.level_min or a.dims[cml][1] < 2:
                break
            dls.append(dl)
            n = m.number_parts(apr, dl)
            x = rng.rand(CIN, n)
            w = rng.randn(NST, COUT, CIN, 3, 3, 3)
            w1 = rng.randn(NST, COUT, CIN, 1, 1, 1)
            go = rng.randn(COUT, n)
            ld = torch.full((1,), dl, dtype=torch.int32)
            xt, got = torch.from_numpy(x)[None], torch.from_numpy(go)[None]
            cpu = lambda t: torch.from_numpy(t).permute(2, 0, 1, 3, 4, 5).contiguous()      # (S,Co,Ci,..) -> (Ci,S,Co,..)
            gpu = lambda t: t.permute(1, 2, 0, 3, 4, 5).contiguous().numpy()
            we = m.restrict_kernel333_forward(cpu(w), L)
            k = "dl%d_" % dl
            out[k + "n"] = n
            out[k + "x"], out[k + "w"], out[k + "w1"], out[k + "go"] = x, w, w1, go
            out[k + "w_expanded"] = gpu(we)
            out[k + "tree"] = m.fill_tree_mean(apr, xt[0], dl).numpy()
            gt = rng.rand(CIN, out[k + "tree"].shape[1])
            out[k + "gt"] = gt
            out[k + "tree_bwd"] = m.fill_tree_mean_backward(apr, xt[0], torch.from_numpy(gt), dl).numpy()
            out[k + "conv333"] = m.convolve333_forward([apr], xt, we, ld)[0].numpy()
            gi, gw = m.convolve333_backward([apr], xt, we, got, ld)
            out[k + "conv333_gi"], out[k + "conv333_gw"] = gi[0].numpy(), gpu(gw)
            out[k + "restrict_bwd"] = gpu(m.restrict_kernel333_backward(gw, NST))
            out[k + "conv111"] = m.convolve111_forward([apr], xt, cpu(w1), ld)[0].numpy()
            gi, gw = m.convolve111_backward([apr], xt, cpu(w1), got, ld)
            out[k + "conv111_gi"], out[k + "conv111_gw"] = gi[0].numpy(), gpu(gw)
            xr = np.round(x * 4) / 4
            out[k + "xr"] = xr
            po, pi = m.maxpool_forward([apr], torch.from_numpy(xr)[None], ld)
            out[k + "pool"], out[k + "pool_idx"] = po[0].numpy(), pi[0].numpy()
            gpo = rng.randn(*out[k + "pool"].shape)
            out[k + "gpo"] = gpo
            out[k + "pool_bwd"] = m.maxpool_backward([apr], torch.from_numpy(gpo)[None], pi, ld)[0].numpy()
            if dl > 0:
                out[k + "up"] = m.upsample_const_forward([apr], xt, ld)[0].numpy()
                gu = rng.randn(CIN, out[k + "up"].shape[1])
                out[k + "gu"] = gu
                out[k + "up_bwd"] = m.upsample_const_backward([apr], torch.from_numpy(gu)[None], ld)[0].numpy()
        out["dls"] = np.array(dls)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "N", a.n_particles, "dls", dls)


if __name__ == "__main__":
    main()
