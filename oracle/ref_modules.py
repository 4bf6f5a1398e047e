"""TEST / BASELINE INFRASTRUCTURE ONLY — CPU operator modules for the timed CPU baseline.

`RefOps` wraps the reference's own CPU operators (module `_apr_ref`, built by build_ref.py from the
reference checkout) in autograd Functions with the constructor / call signatures of the reference's
CPU modules (pyapr/aprnet/conv.py:18-182, pool.py:7-34, upsample.py:7-34), so the same U-Net can be
timed on host cores.  `PortOps` does the same over this repository's restated oracle
(apr_oracle.cpp) and is used when the compiled reference is not present.  Nothing in the product
path imports this file.
"""
import math

import numpy as np
import torch
from torch import nn
from torch.autograd import Function
from torch.nn import init


def make_ops(ref_mod=None):
    """Namespace with APRConv / MaxPool / UpSampleConst running on the CPU.

    `aprs` passed to the modules are lists of handles from `wrap_apr` below."""

    class _Conv(Function):
        @staticmethod
        def forward(ctx, x, w, bias, aprs, level_deltas, ksize):
            ctx.aprs, ctx.ksize, ctx.nst = aprs, ksize, w.shape[0]
            num_levels = max(a.level_max - a.level_min + 1 for a in aprs)
            we = _restrict_fwd(w, num_levels) if ksize == 3 else w
            ctx.save_for_backward(x, we, bias, level_deltas.clone())
            out = _conv_fwd(aprs, x, we, level_deltas, ksize)
            return out if bias is None else out + bias.view(1, -1, 1)

        @staticmethod
        def backward(ctx, go):
            x, we, bias, ld = ctx.saved_tensors
            gi, gwe = _conv_bwd(ctx.aprs, x, we, go.contiguous(), ld, ctx.ksize)
            gw = _restrict_bwd(gwe, ctx.nst) if ctx.ksize == 3 else gwe
            gb = None if bias is None else go.sum(dim=(0, 2))
            return gi, gw, gb, None, None, None

    # weights are kept in the CUDA layout (S, Cout, Cin, k, k, k); the reference CPU code wants
    # (Cin, S, Cout, k, k, k) (pyapr/aprnet/conv.py:164), permuted as its own test does
    # (pyapr/tests/test_aprnet.py:163,177).
    def _to_cpu_layout(w):
        return w.permute(2, 0, 1, 3, 4, 5).contiguous()

    def _from_cpu_layout(w):
        return w.permute(1, 2, 0, 3, 4, 5).contiguous()

    if ref_mod is not None:
        def _restrict_fwd(w, L):
            return _from_cpu_layout(ref_mod.restrict_kernel333_forward(_to_cpu_layout(w), L))

        def _restrict_bwd(gw, S):
            return _from_cpu_layout(ref_mod.restrict_kernel333_backward(_to_cpu_layout(gw), S))

        def _conv_fwd(aprs, x, we, ld, k):
            f = ref_mod.convolve333_forward if k == 3 else ref_mod.convolve111_forward
            return f([a.ref for a in aprs], x, _to_cpu_layout(we), ld)

        def _conv_bwd(aprs, x, we, go, ld, k):
            f = ref_mod.convolve333_backward if k == 3 else ref_mod.convolve111_backward
            gi, gw = f([a.ref for a in aprs], x, _to_cpu_layout(we), go, ld)
            return gi, _from_cpu_layout(gw)

        def _pool_fwd(aprs, x, ld):
            return ref_mod.maxpool_forward([a.ref for a in aprs], x, ld)

        def _pool_bwd(aprs, go, idx, ld):
            return ref_mod.maxpool_backward([a.ref for a in aprs], go, idx, ld)

        def _up_fwd(aprs, x, ld):
            return ref_mod.upsample_const_forward([a.ref for a in aprs], x, ld)

        def _up_bwd(aprs, go, ld):
            return ref_mod.upsample_const_backward([a.ref for a in aprs], go, ld)
    else:
        import apr_oracle as O

        def _batched(fn, aprs, tensors, ld, out_sizes):
            outs = None
            for b, a in enumerate(aprs):
                res = fn(a.orc, [t[b].numpy() for t in tensors], int(ld[b]))
                res = res if isinstance(res, tuple) else (res,)
                if outs is None:
                    outs = [torch.zeros((len(aprs),) + r.shape[:-1] + (out_sizes[i],), dtype=torch.from_numpy(r).dtype)
                            for i, r in enumerate(res)]
                for i, r in enumerate(res):
                    outs[i][b, ..., :r.shape[-1]] = torch.from_numpy(r)
            return outs

        def _restrict_fwd(w, L):
            return torch.from_numpy(O.restrict333_forward(w.detach().numpy(), L))

        def _restrict_bwd(gw, S):
            return torch.from_numpy(O.restrict333_backward(gw.numpy(), S))

        def _conv_fwd(aprs, x, we, ld, k):
            wn = we.detach().numpy()
            f = (lambda o, t, dl: o.conv333_forward(t[0][:, :o.number_parts(dl)], wn, dl)) if k == 3 else \
                (lambda o, t, dl: o.conv111_forward(t[0][:, :o.number_parts(dl)], wn, dl))
            return _batched(f, aprs, [x.detach()], ld, [x.shape[2]])[0]

        def _conv_bwd(aprs, x, we, go, ld, k):
            wn = we.detach().numpy()
            gi = torch.zeros_like(x)
            gw = torch.zeros_like(we)
            for b, a in enumerate(aprs):
                n = a.orc.number_parts(int(ld[b]))
                f = a.orc.conv333_backward if k == 3 else a.orc.conv111_backward
                g1, g2 = f(x[b, :, :n].detach().numpy(), wn, go[b, :, :n].numpy(), int(ld[b]))
                gi[b, :, :n] = torch.from_numpy(g1)
                gw += torch.from_numpy(g2)
            return gi, gw

        def _pool_fwd(aprs, x, ld):
            m = max(a.orc.number_parts(int(ld[b]) + 1) for b, a in enumerate(aprs))
            return _batched(lambda o, t, dl: o.maxpool_forward(t[0][:, :o.number_parts(dl)], dl), aprs, [x.detach()], ld, [m, m])

        def _pool_bwd(aprs, go, idx, ld):
            m = max(a.orc.number_parts(int(ld[b])) for b, a in enumerate(aprs))
            f = lambda o, t, dl: o.maxpool_backward(t[0][:, :o.number_parts(dl + 1)], t[1][:, :o.number_parts(dl + 1)], dl)
            return _batched(f, aprs, [go, idx], ld, [m])[0]

        def _up_fwd(aprs, x, ld):
            m = max(a.orc.number_parts(int(ld[b]) - 1) for b, a in enumerate(aprs))
            return _batched(lambda o, t, dl: o.upsample_forward(t[0][:, :o.number_parts(dl)], dl), aprs, [x.detach()], ld, [m])[0]

        def _up_bwd(aprs, go, ld):
            m = max(a.orc.number_parts(int(ld[b])) for b, a in enumerate(aprs))
            return _batched(lambda o, t, dl: o.upsample_backward(t[0][:, :o.number_parts(dl - 1)], dl), aprs, [go], ld, [m])[0]

    class _Pool(Function):
        @staticmethod
        def forward(ctx, x, aprs, ld, inc):
            out, idx = _pool_fwd(aprs, x, ld)
            ctx.aprs = aprs
            ctx.save_for_backward(idx, ld.clone())
            if inc:
                ld.add_(1)
            return out

        @staticmethod
        def backward(ctx, go):
            idx, ld = ctx.saved_tensors
            return _pool_bwd(ctx.aprs, go.contiguous(), idx, ld), None, None, None

    class _Up(Function):
        @staticmethod
        def forward(ctx, x, aprs, ld, dec):
            ctx.aprs = aprs
            ctx.save_for_backward(ld.clone())
            out = _up_fwd(aprs, x, ld)
            if dec:
                ld.sub_(1)
            return out

        @staticmethod
        def backward(ctx, go):
            ld, = ctx.saved_tensors
            return _up_bwd(ctx.aprs, go.contiguous(), ld), None, None, None

    class APRConv(nn.Module):
        def __init__(self, in_channels, out_channels, nstencils=1, kernel_size=(3, 3, 3), bias=True):
            super().__init__()
            self.k = kernel_size[0]
            self.weight = nn.Parameter(torch.empty(nstencils, out_channels, in_channels, *kernel_size))
            self.bias = nn.Parameter(torch.empty(out_channels)) if bias else None
            init.kaiming_uniform_(self.weight, a=math.sqrt(5))
            if self.bias is not None:
                fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
                init.uniform_(self.bias, -1 / math.sqrt(fan_in), 1 / math.sqrt(fan_in))

        def forward(self, x, aprs, level_deltas):
            return _Conv.apply(x, self.weight, self.bias, aprs, level_deltas, self.k)

    class MaxPool(nn.Module):
        def __init__(self):
            super().__init__()
            self.increment_level_deltas = True

        def forward(self, x, aprs, level_deltas):
            return _Pool.apply(x, aprs, level_deltas, self.increment_level_deltas)

    class UpSampleConst(nn.Module):
        def __init__(self):
            super().__init__()
            self.decrement_level_deltas = True

        def forward(self, x, aprs, level_deltas):
            return _Up.apply(x, aprs, level_deltas, self.decrement_level_deltas)

    class Ops:
        pass

    ops = Ops()
    ops.APRConv, ops.MaxPool, ops.UpSampleConst = APRConv, MaxPool, UpSampleConst
    ops.kind = "reference" if ref_mod is not None else "port"
    return ops


class CpuApr:
    """One APR for the CPU modules: carries the reference stand-in object and/or the oracle handle."""

    def __init__(self, arrays, ref_mod=None):
        self.level_min, self.level_max = int(arrays.level_min), int(arrays.level_max)
        self.arrays = arrays
        if ref_mod is not None:
            import ref as _ref
            self.ref = _ref.make_apr(ref_mod, arrays)
        else:
            import apr_oracle as O
            self.orc = O.OracleAPR(arrays)
