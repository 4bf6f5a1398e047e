#!/usr/bin/env python
"""Benchmark of the particle-domain CNN hot path: APR U-Net forward + backward (+ SGD step).

    python bench.py --gpus N --steps K --warmup W            # this implementation (CUDA, one rank per GPU)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU operators on host cores

One step = one training pass of the 4-level APR U-Net (base 32 channels, 2 convs per level, GroupNorm,
ReLU, max-pool down / up-sample + concat up, 2 classes, cross-entropy against blob-interior labels)
over one synthetic APR per GPU.  Inputs are seeded synthetic blob volumes (no dataset ships with the
reference); metric = particles per second, summed over GPUs (weak scaling: one APR of the configured
size per GPU, gradients all-reduced over NCCL).  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "apr-cnn_b200"))

import numpy as np
import torch


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--volume", default="", help="z,x,y of the synthetic image (default: the headline config)")
    ap.add_argument("--blobs", type=int, default=0)
    ap.add_argument("--base", type=int, default=32)
    ap.add_argument("--depth", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["f32", "bf16"],
                    help="arithmetic of the 3x3x3 convolutions: exact fp32 CUDA-core kernels, or bf16 tensor-core contraction with fp32 accumulation")
    ap.add_argument("--cpu-sample", default="64,128,128", help="volume of the bounded CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--config", type=int, default=3, choices=[2, 3, 4, 5],
                    help="which configuration of BASELINE.json: 3 = U-Net training step (default, the headline), 2 = forward-only block stack "
                         "(conv 1->32, pool, conv 32->64, up-sample, 1x1x1 conv 64->2; fp32) on the 256x512x512 APR, 4 = batch inference over "
                         "64 independent APRs, 5 = APRConv channel sweep (one JSON line per shape, stencil and dtype)")
    ap.add_argument("--layer", default="", help="cin,cout,level_delta[,ksize]: time ONE APRConv layer (forward + backward) instead of the U-Net")
    ap.add_argument("--batch-inference", type=int, default=0,
                    help="configs[3] of BASELINE.json: forward-only U-Net over this many independent APRs (256^3 images, 50-400 blobs), "
                         "split over the ranks with no collective; reports aggregate particles/s")
    ap.add_argument("--shard", default="zslab", choices=["zslab", "replica"],
                    help="with more than one GPU: 'zslab' cuts the ONE configured APR into z-slabs, one per GPU, with halo exchange "
                         "before every 3x3x3 layer (strong scaling); 'replica' gives every GPU its own APR of the configured size "
                         "(weak scaling, gradient all-reduce only)")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the timed region run one more step between cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    a = ap.parse_args()
    a.dtype_given = a.dtype if any(x == "--dtype" or x.startswith("--dtype=") for x in sys.argv[1:]) else None
    return a


HEADLINE_VOLUME = (512, 1024, 1024)      # configs[2] of BASELINE.json: 1024x1024x512 image, 5000 blobs
HEADLINE_BLOBS = 5000


def blob_count(volume, blobs):
    if blobs > 0:
        return blobs
    dens = HEADLINE_BLOBS / float(np.prod(HEADLINE_VOLUME))
    return max(4, int(round(dens * float(np.prod(volume)))))


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------
# workload construction
# ---------------------------------------------------------------------------------------------
_SYNTHETIC = None


def load_synthetic():
    """`pyapr/synthetic.py` as a stand-alone module: pure torch / numpy code, loaded by path so that the
    reference arm never imports the package (and with it the product's native library)."""
    global _SYNTHETIC
    if _SYNTHETIC is None:
        import importlib.util
        spec = importlib.util.spec_from_file_location("aprnet_bench_synthetic", os.path.join(ROOT, "apr-cnn_b200", "pyapr", "synthetic.py"))
        _SYNTHETIC = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = _SYNTHETIC
        spec.loader.exec_module(_SYNTHETIC)
    return _SYNTHETIC


def make_inputs(volume, blobs, seed, device):
    """Seeded blob volume -> APR arrays, particle intensities (input channel) and labels."""
    synthetic = load_synthetic()
    img = synthetic.blob_image(volume, blobs, seed, device=device)
    arrays = synthetic.apr_from_image(img)
    feat = synthetic.sample_particles_from_image(img, arrays)
    del img
    labels = (feat > 300.0).astype(np.int64)          # blob interiors: well above background 100 + noise
    feat = (feat - 100.0) / 500.0
    return arrays, feat, labels


class Clocks(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.gpu_index = gpu_index
        self.samples = []
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                f = [s.strip() for s in line.split(",")]
                if len(f) >= 9:
                    self.samples.append(f)
        except Exception:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=2)
        sm = sorted(float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def unet_conv_layers(base, depth):
    """(kind, cin, cout, level_delta) of every convolution of the U-Net, forward order."""
    w = [base * 2 ** i for i in range(depth + 1)]
    layers = [("333", 1, w[0], 0), ("333", w[0], w[0], 0)]
    for i in range(depth):
        layers += [("333", w[i], w[i + 1], i + 1), ("333", w[i + 1], w[i + 1], i + 1)]
    for i in reversed(range(depth)):
        layers += [("111", w[i + 1], w[i + 1] // 2, i + 1), ("333", w[i + 1], w[i], i), ("333", w[i], w[i], i)]
    layers.append(("111", w[0], 2, 0))
    return layers


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture per kernel family on the 64->64
# layer at level_delta 1 of a 256x512x512 volume, 1.86 M locations) divided by the algorithmic bytes of the
# same operator call.  Every operand of these kernels is streamed, so traffic scales with the locations.
NCU_TRAFFIC_RATIO = {"conv333_tc_dw": 2.11, "conv333_tc_fwd": 1.36, "conv333_tc_bwd_gather": 1.29}


GN_BYTES = {"groupnorm_stats": 4.0, "groupnorm_relu_apply": 8.0, "groupnorm_bwd_reduce": 8.0, "groupnorm_bwd_apply": 12.0}


def kernel_table(prof, steps, nparts, ntree, peaks, layers, bf16, fma_tflops=None):
    """One row per profiled kernel name: launches, time per step, algorithmic work per step and the fraction of the
    roofline that bounds it.  3x3x3 kernels carry their shape in the name; the streaming kernels are summed over the
    layers that call them.  Per operator call: flops = 54 * cin * cout * N(dl); bytes = (e * cin + 4 * cout + 2) * N
    + e * cin * T for the 3x3x3 passes (e = 2 on the bf16 path, 4 on fp32); 4 * (cin + cout) * N for a 1x1x1 pass (forward,
    input gradient or weight gradient);
    4 * c * (N + 2 T) + 36 T for a tree fill (children read, node written and read by its parent, child table) and
    4 * c * (2 N + 2 T) + 36 T for its adjoint; 6 * c * rows for a packing pass; 4 / 8 / 8 / 12 bytes per element for
    the four GroupNorm passes.  Pooling / up-sampling (part kernel, part strided copy) and the per-(target, tap) sums of the
    cross-level input gradient are listed with their time only."""
    e_in = 2.0 if bf16 else 4.0
    ridge = peaks["tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
    c333 = [(ci, co, dl) for k, ci, co, dl in layers if k == "333"]
    c111 = [(ci, co, dl) for k, ci, co, dl in layers if k == "111"]
    gn = [(co, dl) for k, ci, co, dl in layers[:-1]]                          # every convolution but the head is followed by GroupNorm
    first = c333[0]
    agg = {
        "tree_mean_fwd": sum(4.0 * ci * (nparts[dl] + 2 * ntree[dl]) + 36.0 * ntree[dl] for ci, co, dl in c333),
        "tree_mean_bwd": sum(4.0 * ci * (2 * nparts[dl] + 2 * ntree[dl]) + 36.0 * ntree[dl] for ci, co, dl in c333 if (ci, co, dl) != first),
        "pack_rows_bf16": sum(6.0 * ci * (nparts[dl] + ntree[dl]) for ci, co, dl in c333 if ci > 4) + sum(6.0 * co * nparts[dl] for ci, co, dl in c333 if (ci, co, dl) != first),
    }
    # 1x1x1 passes: the tensor-core forward / input-gradient kernel carries its shape in the name (conv111_tc:ci..:co..:dl..,
    # channel roles swapped in the input gradient); the CUDA-core kernel "conv111" ran the layers no such name covers.
    # The weight gradient runs under one name in either arithmetic.
    tc111 = set()
    for name in prof:
        parts = name.split(":")
        if parts[0] == "conv111_tc" and len(parts) == 4:
            a, b, d = int(parts[1][2:]), int(parts[2][2:]), int(parts[3][2:])
            tc111.update([(a, b, d), (b, a, d)])
    agg["conv111"] = sum(2 * 4.0 * (ci + co) * nparts[dl] for ci, co, dl in c111 if (ci, co, dl) not in tc111)
    dw111 = sum(4.0 * (ci + co) * nparts[dl] for ci, co, dl in c111)
    if "conv111_tc_dw" in prof and "conv111_dw" in prof:
        dw111 = None                                                   # mixed: no per-name split
    agg["conv111_dw"] = agg["conv111_tc_dw"] = dw111
    for name, bpe in GN_BYTES.items():
        agg[name] = sum(bpe * c * nparts[dl] for c, dl in gn)
    rows = []
    for name, (calls, ms) in sorted(prof.items(), key=lambda kv: -kv[1][1]):
        parts = name.split(":")
        row = {"kernel": name, "launches_per_step": calls / steps, "ms_per_step": ms / steps}
        flops = byts = None
        if len(parts) == 4 and parts[1].startswith("ci"):
            ci, co, dl = int(parts[1][2:]), int(parts[2][2:]), int(parts[3][2:])
            n_ops = max(1, sum(1 for s_ in c333 if s_ == (ci, co, dl)))
            fam = parts[0]
            if fam in ("conv333_tc_fwd", "conv333_tc_bwd_gather", "conv333_tc_dw", "conv333_fwd", "conv333_bwd_input", "conv333_dw",
                       "conv333_small_fwd", "conv333_small_dw"):
                e = 4.0 if fam.startswith("conv333_small") else e_in
                flops = n_ops * 54.0 * ci * co * nparts[dl]
                byts = n_ops * ((e * ci + 4.0 * co + 2.0) * nparts[dl] + e * ci * ntree[dl])
            elif fam == "conv111_tc":
                byts = 4.0 * (ci + co) * nparts[dl] * (calls / steps)
        elif name in agg:
            byts = agg[name]
        if byts:
            sec = ms / steps * 1e-3
            tensor_peak = peaks["tflops"] if (bf16 and not parts[0].startswith("conv333_small")) else fma_tflops
            if flops and tensor_peak and flops / byts > tensor_peak * 1e12 / (peaks["hbm_gbs"] * 1e9):
                row.update(bound="tensor" if tensor_peak == peaks["tflops"] else "fp32_fma", achieved=flops / sec / 1e12, peak=tensor_peak,
                           unit="TFLOP/s", frac=flops / sec / 1e12 / tensor_peak)
            else:
                row.update(bound="hbm", achieved=byts / sec / 1e9, peak=peaks["hbm_gbs"], unit="GB/s", frac=byts / sec / 1e9 / peaks["hbm_gbs"])
            row.update(algorithmic_flops_per_step=flops, algorithmic_bytes_per_step=byts)
        rows.append(row)
    return rows


def roofline_from_profile(prof, steps, nparts, ntree, peaks, layers, bf16):
    """Roofline entry of the convolution kernel that took the most time in the timed region.

    Kernel names carry their shape: `conv333_tc_dw:ci32:co32:dl0`.  All shapes of one kernel function
    (the part of the name before the first colon) form one family; the family with the largest total
    time is reported, its launches summed.  Algorithmic work of one 3x3x3 operator call on one APR:
    flops = 54 * cin * cout * N(dl) for the forward pass, the same-level input gradient and the weight
    gradient alike; bytes = (e_in * cin + 4 * cout) * N + 2 * N + e_in * cin * T, with e_in = 2 on the
    bf16 path (packed rows) and 4 on the fp32 path, N the particles of that level_delta, T the tree
    nodes, 2 * N the y coordinates of the access structure.  The bound is the tensor pipe when
    flops/bytes exceeds the ridge of the measured peaks, HBM otherwise."""
    if not prof:
        return None
    total_ms = sum(v[1] for v in prof.values())
    fams = {}
    for name, (calls, ms) in prof.items():
        parts = name.split(":")
        if len(parts) == 4 and parts[0].startswith("conv333") and parts[0] != "conv333_tc_edge" and parts[1].startswith("ci"):
            fams.setdefault(parts[0], []).append((int(parts[1][2:]), int(parts[2][2:]), int(parts[3][2:]), calls, ms))
    if not fams:
        name, (calls, ms) = max(prof.items(), key=lambda kv: kv[1][1])
        return {"kernel": name, "share_of_profiled": ms / total_ms}
    fam, rows = max(fams.items(), key=lambda kv: sum(r[4] for r in kv[1]))
    e_in = 2.0 if bf16 else 4.0
    flops = byts = ms_sum = 0.0
    launches = ops = 0
    for cin, cout, dl, calls, ms in rows:
        # the gather kernels run once per operator call; the weight-gradient kernels run once per level
        n_ops = max(1, sum(1 for k, ci, co, d in layers if k == "333" and (ci, co, d) == (cin, cout, dl))) * steps \
            if fam in ("conv333_dw", "conv333_tc_dw") else calls
        n, t = nparts[dl], ntree[dl]
        flops += n_ops * 54.0 * cin * cout * n
        byts += n_ops * ((e_in * cin + 4.0 * cout + 2.0) * n + e_in * cin * t)
        ms_sum += ms
        launches += calls
        ops += n_ops
    sec = ms_sum * 1e-3
    ridge = peaks["tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
    rf = {"kernel": fam, "shapes": len(rows), "launches": launches, "operator_calls": ops,
          "share_of_profiled": ms_sum / total_ms, "avg_ms": ms_sum / max(1, launches)}
    if flops / byts > ridge:
        ach = flops / sec / 1e12
        rf.update(bound="tensor", achieved=ach, peak=peaks["tflops"], unit="TFLOP/s", frac=ach / peaks["tflops"])
    else:
        ach = byts / sec / 1e9
        rf.update(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
    rf.update(algorithmic_flops_per_launch=flops / max(1, launches), algorithmic_bytes_per_launch=byts / max(1, launches),
              hbm_gbs_at_algorithmic_bytes=byts / sec / 1e9, peak_source=peaks["source"],
              traffic=(byts / max(1, launches)) * NCU_TRAFFIC_RATIO[fam] if fam in NCU_TRAFFIC_RATIO else None,
              traffic_source="algorithmic bytes x the dram__bytes ratio of an ncu capture of this kernel on the 64->64 layer at level_delta 1 of a "
                             "256x512x512 volume (1.86 M locations), scaled by locations" if fam in NCU_TRAFFIC_RATIO else None)
    return rf


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU operators on host cores (bounded sample)
# ---------------------------------------------------------------------------------------------
def run_cpu(args, steps, warmup, stack=False):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref as ref_loader
    import ref_modules
    from apr_unet import APRUNet
    ref_mod = ref_loader.load()
    if ref_mod is None:
        import apr_oracle
        apr_oracle.build()
    ops = ref_modules.make_ops(ref_mod)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if ref_mod is not None:
        ref_mod.set_num_threads(cores)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    vol = tuple(int(v) for v in args.cpu_sample.split(","))
    blobs = blob_count(vol, 0)
    arrays, feat, labels = make_inputs(vol, blobs, 3000, "cpu")
    apr = ref_modules.CpuApr(arrays, ref_mod)
    x = torch.from_numpy(feat)[None, None].contiguous()
    y = torch.from_numpy(labels)[None]
    if stack:
        _, forward = build_stack(ops)

        def step():
            with torch.no_grad():
                return float(forward(x, [apr]).sum())
    else:
        torch.manual_seed(7)
        model = APRUNet(ops, 1, 2, depth=args.depth, n_filters_base=args.base)
        opt = torch.optim.SGD(model.parameters(), lr=1e-3)

        def step():
            opt.zero_grad(set_to_none=True)
            out = model(x, [apr])
            loss = torch.nn.functional.cross_entropy(out, y)
            loss.backward()
            opt.step()
            return float(loss.detach())

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    n = arrays.n_particles
    return {"value": n / dt, "unit": "particles/s", "cores": cores, "kind": ops.kind,
            "sample": "%s, fp32, one APR from a %dx%dx%d (z,x,y) blob volume with %d blobs: %d particles, %.2f s/step, %d timed step(s) after %d warm-up"
                      % ("block stack forward" if stack else "U-Net fwd+bwd+SGD", vol[0], vol[1], vol[2], blobs, n, dt, steps, warmup),
            "ms_per_step": dt * 1e3, "particles": n}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the b200 arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    from apr_unet import APRUNet
    from pyapr.sharding import allreduce_gradients, zslab_plan

    C.set_conv_precision("bf16" if args.dtype == "bf16" else "fp32")
    volume = tuple(int(v) for v in args.volume.split(",")) if args.volume else HEADLINE_VOLUME
    blobs = blob_count(volume, args.blobs)
    zslab = world > 1 and args.shard == "zslab"
    t_setup = time.perf_counter()
    # z-slabs: every rank builds the same APR (same seed) and keeps its slab; replicas: one APR per rank
    arrays, feat, labels = make_inputs(volume, blobs, 3000 + (0 if zslab else rank), dev)
    n_global = arrays.n_particles
    shard = None
    if zslab:
        # the plans are computed independently on every rank: they only pair up if all ranks hold the same structure
        sig = torch.tensor([arrays.n_particles, arrays.n_tree, int(np.asarray(arrays.row_ptr, dtype=np.int64).sum() % (1 << 40)),
                            int(np.asarray(arrays.y, dtype=np.int64).sum() % (1 << 40))], dtype=torch.int64, device=dev)
        sigs = [torch.zeros_like(sig) for _ in range(world)]
        dist.all_gather(sigs, sig)
        if any(not torch.equal(s_, sig) for s_ in sigs):
            raise RuntimeError("z-slab sharding: the ranks built different APRs from the same seed; refusing to exchange halos")
        from pyapr.aprnet.cuda.sharded import Shard, make_ops, sharded_cross_entropy
        plan = zslab_plan(arrays, rank, world, max_level_delta=args.depth)
        feat, labels = feat[plan.l2g_particles], labels[plan.l2g_particles]
        arrays = plan.local
    apr = pyapr.apr_from_arrays(arrays, "bench")
    apr.init_cuda()
    if zslab:
        shard = Shard(plan, dev)
        ops = make_ops(shard)
    nparts = [int(pyapr.aprnet.utils.number_particles(apr, dl)) for dl in range(args.depth + 1)]
    o_tree = []
    for dl in range(args.depth + 1):
        apr.plan(dl)
        cml = arrays.level_max - dl
        r = sum(arrays.dims[l][0] * arrays.dims[l][1] for l in range(0, cml))
        o_tree.append(int(arrays.tree_row_ptr[r]))
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup

    torch.manual_seed(7)
    model = APRUNet(ops, 1, 2, depth=args.depth, n_filters_base=args.base).to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    params = [p for p in model.parameters()]
    x_host = torch.from_numpy(feat)[None, None].contiguous().pin_memory()
    y_host = torch.from_numpy(labels)[None].contiguous().pin_memory()
    x_dev, y_dev = x_host.to(dev), y_host.to(dev)
    n_local = n_global if not zslab else int(plan.owned_particles.sum())

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        out = model(x, [apr])
        if zslab:
            loss, loss_all = sharded_cross_entropy(out, y, shard)
            loss.backward()
            allreduce_gradients(params, world, average=False)      # every rank holds a partial sum of the same sample
            opt.step()
            return loss_all
        loss = torch.nn.functional.cross_entropy(out, y)
        loss.backward()
        allreduce_gradients(params, world)
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(x_dev, y_dev)
    barrier()

    # ---- timed region: inputs resident in HBM --------------------------------------------------
    clocks = Clocks(local_rank) if rank == 0 else None
    if clocks:
        clocks.start()
        time.sleep(0.3)
    C.profile_read()
    C.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step(x_dev, y_dev)
    e1.record()
    barrier()
    C.profile_enable(False)
    ms = e0.elapsed_time(e1)
    prof = C.profile_read()
    clock_rec = clocks.stop() if clocks else None
    loss_val = float(loss.detach())

    if args.profile_step:
        barrier()
        torch.cuda.profiler.start()
        step(x_dev, y_dev)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()

    # ---- end-to-end: host buffers in, loss out, every step --------------------------------------
    e2e = None
    if not args.no_e2e:
        barrier()
        e0.record()
        for _ in range(args.steps):
            xd = x_host.to(dev, non_blocking=True)
            yd = y_host.to(dev, non_blocking=True)
            lv = step(xd, yd).item()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    h2d_local = float(x_host.numel() * 4 + y_host.numel() * 8)
    t = torch.tensor([ms, e2e_ms if not args.no_e2e else 0.0, float(n_local), h2d_local], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, e2e_ms_all, n_total, h2d_total = float(tmax[0]), float(tmax[1]), float(tsum[2]), float(tsum[3])
    else:
        ms, e2e_ms_all, n_total, h2d_total = float(t[0]), float(t[1]), float(t[2]), float(t[3])

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return None
    peaks = load_peaks()
    ms_per_step = ms / args.steps
    launches = int(sum(v[0] for v in prof.values()))
    out = {
        "metric": "APR U-Net fwd+bwd particles/s", "value": n_total / (ms_per_step * 1e-3), "unit": "particles/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if zslab else "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": "4-level APR U-Net (base %d, 2 convs/level, GroupNorm, ReLU, 2 classes) fwd+bwd+SGD on %s from a "
                               "seeded %dx%dx%d (z,x,y) uint16 blob volume, %d blobs"
                               % (args.base, "ONE APR cut into %d z-slabs" % world if zslab else "one APR per GPU", volume[0], volume[1], volume[2], blobs),
                   "particles_total": int(n_total), "particles_rank0": n_local, "particles_by_level_delta_rank0": nparts,
                   "tree_nodes_by_level_delta_rank0": o_tree,
                   "parallelism": ("z-slab sharding of one APR: slab boundaries (voxels) %s, halo rows exchanged point-to-point (NCCL send/recv) before "
                                   "every 3x3x3 layer and back in its backward pass, GroupNorm sums and weight gradients all-reduced" % (plan.cuts,)) if zslab
                                  else ("one APR replica per GPU, gradient all-reduce (NCCL)" if world > 1 else "single GPU"),
                   "l2": "inputs larger than L2 (activations are GBs per layer)", "setup_s": t_setup, "loss": loss_val},
        "gpu_launches": launches,
        "max_memory_gb": torch.cuda.max_memory_allocated() / 1e9, "apr_table_gb": apr.cuda_device_bytes() / 1e9,
        "clocks": clock_rec,
    }
    if e2e_ms_all:
        out["e2e"] = {"value": n_total / (e2e_ms_all / args.steps * 1e-3), "unit": "particles/s",
                      "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": 4 * world}
    layers = unet_conv_layers(args.base, args.depth)
    fma = float(C.measure_fp32_fma_tflops(5))
    out["roofline"] = roofline_from_profile(prof, args.steps, nparts, o_tree, peaks, layers, args.dtype == "bf16")
    out["roofline_by_shape"] = kernel_table(prof, args.steps, nparts, o_tree, peaks, layers, args.dtype == "bf16", fma)
    out["fp32_fma_tflops_measured"] = fma
    if world == 1 and not args.no_cpu_baseline:
        cb = run_cpu(args, 3, 1)
        out["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if world > 1:
        dist.destroy_process_group()
    return out



# ---------------------------------------------------------------------------------------------
# batch inference over independent APRs (configs[3] of BASELINE.json): no data-path collective
# ---------------------------------------------------------------------------------------------
def run_batch_inference(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    from apr_unet import APRUNet
    from pyapr.sharding import shard_indices
    C.set_conv_precision("bf16" if args.dtype == "bf16" else "fp32")
    torch.manual_seed(7)
    model = APRUNet(ops, 1, 2, depth=args.depth, n_filters_base=args.base).to(dev).eval()
    rng = np.random.RandomState(4000)
    blob_counts = rng.randint(50, 401, size=args.batch_inference)
    mine = shard_indices(args.batch_inference, rank, world)
    items = []
    for i in mine:                                   # image i -> rank i mod world; nothing is exchanged
        arrays, feat, _ = make_inputs((256, 256, 256), int(blob_counts[i]), 4000 + int(i), dev)
        apr = pyapr.apr_from_arrays(arrays, "img%d" % i)
        apr.init_cuda()
        for dl in range(args.depth + 1):
            apr.plan(dl)
        items.append((apr, torch.from_numpy(feat)[None, None].contiguous().to(dev), arrays.n_particles))
    n_local = sum(it[2] for it in items)

    def sweep():
        with torch.no_grad():
            for apr, x, _ in items:
                model(x, [apr])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup)):
        sweep()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        sweep()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1), float(n_local)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax, tsum = t.clone(), t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, n_total = float(tmax[0]), float(tsum[1])
        dist.destroy_process_group()
    else:
        ms, n_total = float(t[0]), float(t[1])
    if rank != 0:
        return None
    ms_per_sweep = ms / args.steps
    return {"metric": "APR U-Net forward particles/s (batch inference)", "value": n_total / (ms_per_sweep * 1e-3), "unit": "particles/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(1, args.warmup), "ms_per_step": ms_per_sweep, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": "forward-only 4-level APR U-Net (base %d) over %d independent APRs from seeded 256x256x256 blob volumes "
                                   "(50-400 blobs each), image i on rank i mod %d, no collective" % (args.base, args.batch_inference, world),
                       "particles_total": int(n_total)}}


# ---------------------------------------------------------------------------------------------
# single-layer mode (APRConv channel sweep: configs[4] of BASELINE.json)
# ---------------------------------------------------------------------------------------------
_LAYER_APR = {}


def run_layer(args, peaks=None):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    f = [int(v) for v in args.layer.split(",")]
    cin, cout, dl = f[0], f[1], f[2]
    k = f[3] if len(f) > 3 else 3
    C.set_conv_precision("bf16" if args.dtype == "bf16" else "fp32")
    volume = tuple(int(v) for v in args.volume.split(",")) if args.volume else (256, 512, 512)
    blobs = blob_count(volume, args.blobs)
    if (volume, blobs) not in _LAYER_APR:
        arrays, _, _ = make_inputs(volume, blobs, 2000, dev)
        apr = pyapr.apr_from_arrays(arrays, "layer")
        apr.init_cuda()
        _LAYER_APR.clear()
        _LAYER_APR[(volume, blobs)] = (arrays, apr)
    arrays, apr = _LAYER_APR[(volume, blobs)]
    apr.plan(dl)
    n = int(pyapr.aprnet.utils.number_particles(apr, dl))
    cml = arrays.level_max - dl
    t = int(arrays.tree_row_ptr[sum(arrays.dims[l][0] * arrays.dims[l][1] for l in range(0, cml))])
    torch.manual_seed(7)
    conv = ops.APRConv(cin, cout, nstencils=2, kernel_size=(k, k, k), bias=False).to(dev)
    x_host = torch.rand(1, cin, n).pin_memory()
    x = x_host.to(dev).requires_grad_(True)
    go = torch.randn(1, cout, n, device=dev)
    ld = torch.full((1,), dl, dtype=torch.int32)

    def step(xx):
        xx.grad = None
        conv.weight.grad = None
        conv(xx, [apr], ld).backward(go)

    for _ in range(max(3, args.warmup)):
        step(x)
    torch.cuda.synchronize()
    C.profile_read()
    C.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(x)
    e1.record()
    torch.cuda.synchronize()
    C.profile_enable(False)
    prof = C.profile_read()
    if args.profile_step:
        torch.cuda.profiler.start()
        step(x)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    e0.record()
    for _ in range(args.steps):
        xe = x_host.to(dev, non_blocking=True).requires_grad_(True)
        step(xe)
        chk = float(conv.weight.grad.sum().item())
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    peaks = peaks or load_peaks()
    bf16 = args.dtype == "bf16" and k == 3
    fma = float(C.measure_fp32_fma_tflops(3))
    flops = (54.0 if k == 3 else 2.0) * cin * cout * n
    e_in = 2.0 if bf16 and cin > 4 else 4.0
    byts = (e_in * cin + 4.0 * cout + 2.0) * n + (e_in * cin * t if k == 3 else 0.0)
    # the three passes (forward, input gradient, weight gradient) together against the roofline of one pass x 3
    conv_ms = sum(v[1] for kk, v in prof.items() if kk.startswith(("conv333", "conv111"))) / args.steps
    peak_c = peaks["tflops"] if bf16 and cin > 4 else fma
    if flops / byts > peak_c * 1e12 / (peaks["hbm_gbs"] * 1e9):
        ach = 3 * flops / (conv_ms * 1e-3) / 1e12
        rf = {"bound": "tensor" if peak_c == peaks["tflops"] else "fp32_fma", "achieved": ach, "peak": peak_c, "unit": "TFLOP/s", "frac": ach / peak_c}
    else:
        ach = 3 * byts / (conv_ms * 1e-3) / 1e9
        rf = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
    rf.update(kernel="convolution kernels of the three passes", ms=conv_ms, traffic=None, peak_source=peaks["source"])
    out = {"metric": "APRConv layer fwd+bwd particles/s", "value": n / (ms * 1e-3), "unit": "particles/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": args.dtype if k == 3 else "f32", "data": "synthetic",
           "config": {"workload": "APRConv %dx%dx%d %d->%d at level_delta %d, forward + backward, %dx%dx%d volume" % (k, k, k, cin, cout, dl, *volume),
                      "particles": n, "tree_nodes": t, "l2": "inputs larger than L2" if (cin + cout) * n * 4 > 126e6 else "L2 not flushed: operands of this narrow layer fit L2"},
           "gpu_launches": int(sum(v[0] for v in prof.values())),
           "e2e": {"value": n / (e2e_ms * 1e-3), "unit": "particles/s", "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": 4},
           "roofline": rf, "fp32_fma_tflops_measured": fma,
           "algorithmic": {"flops_per_pass": flops, "bytes_per_pass": byts,
                           "tensor_roofline_ms_per_pass": flops / (peaks["tflops"] * 1e12) * 1e3,
                           "hbm_roofline_ms_per_pass": byts / (peaks["hbm_gbs"] * 1e9) * 1e3},
           "kernels": {kk: {"launches": v[0] / args.steps, "ms": v[1] / args.steps} for kk, v in sorted(prof.items(), key=lambda kv: -kv[1][1])}}
    del x, go, conv
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------
# forward-only block stack (configs[1] of BASELINE.json)
# ---------------------------------------------------------------------------------------------
STACK_LAYERS = [("333", 1, 32, 0), ("333", 32, 64, 1), ("111", 64, 2, 0)]


def build_stack(ops):
    """conv3x3x3 1->32 @dl0 -> MaxPool -> conv3x3x3 32->64 @dl1 -> UpSampleConst -> conv1x1x1 64->2 @dl0, one stencil, biases on."""
    torch.manual_seed(7)
    mods = torch.nn.ModuleList([ops.APRConv(1, 32, nstencils=1, kernel_size=(3, 3, 3)), ops.MaxPool(),
                                ops.APRConv(32, 64, nstencils=1, kernel_size=(3, 3, 3)), ops.UpSampleConst(),
                                ops.APRConv(64, 2, nstencils=1, kernel_size=(1, 1, 1))])

    def forward(x, aprs):
        ld = torch.zeros(len(aprs), dtype=torch.int32)
        for m in mods:
            x = m(x, aprs, ld)
        return x
    return mods, forward


def run_block_stack(args):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    import pyapr
    from pyapr.aprnet import cuda as ops
    from _pyaprwrapper.aprnet import cuda as C
    dtype = "f32" if args.dtype_given is None else args.dtype
    C.set_conv_precision("bf16" if dtype == "bf16" else "fp32")
    volume = tuple(int(v) for v in args.volume.split(",")) if args.volume else (256, 512, 512)
    blobs = blob_count(volume, args.blobs)
    arrays, feat, _ = make_inputs(volume, blobs, 2000, dev)
    apr = pyapr.apr_from_arrays(arrays, "stack")
    apr.init_cuda()
    nparts, o_tree = [], []
    for dl in (0, 1):
        apr.plan(dl)
        nparts.append(int(pyapr.aprnet.utils.number_particles(apr, dl)))
        cml = arrays.level_max - dl
        o_tree.append(int(arrays.tree_row_ptr[sum(arrays.dims[l][0] * arrays.dims[l][1] for l in range(0, cml))]))
    mods, forward = build_stack(ops)
    mods.to(dev)
    x_host = torch.from_numpy(feat)[None, None].contiguous().pin_memory()
    x_dev = x_host.to(dev)
    n = arrays.n_particles

    def step(x):
        with torch.no_grad():
            return forward(x, [apr])

    for _ in range(max(3, args.warmup)):
        step(x_dev)
    torch.cuda.synchronize()
    clocks = Clocks(0)
    clocks.start()
    time.sleep(0.3)
    C.profile_read()
    C.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step(x_dev)
    e1.record()
    torch.cuda.synchronize()
    C.profile_enable(False)
    prof = C.profile_read()
    ms = e0.elapsed_time(e1) / args.steps
    e0.record()
    for _ in range(args.steps):
        chk = float(step(x_host.to(dev, non_blocking=True)).sum().item())
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    clock_rec = clocks.stop()
    peaks = load_peaks()
    fma = float(C.measure_fp32_fma_tflops(5))
    table = kernel_table(prof, args.steps, nparts, o_tree, peaks, STACK_LAYERS, dtype == "bf16", fma)
    top = next((r for r in table if "frac" in r), None)
    res = {"metric": "APR block stack forward particles/s", "value": n / (ms * 1e-3), "unit": "particles/s", "n_gpus": 1, "steps": args.steps,
           "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype,
           "data": "synthetic",
           "config": {"workload": "forward-only block stack conv3x3x3 1->32, MaxPool, conv3x3x3 32->64, UpSampleConst, conv1x1x1 64->2 on one APR from a "
                                  "seeded %dx%dx%d (z,x,y) uint16 blob volume, %d blobs" % (volume[0], volume[1], volume[2], blobs),
                      "particles": n, "particles_by_level_delta": nparts, "l2": "inputs larger than L2", "checksum": chk},
           "gpu_launches": int(sum(v[0] for v in prof.values())), "clocks": clock_rec,
           "e2e": {"value": n / (e2e_ms * 1e-3), "unit": "particles/s", "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": 4},
           "roofline": dict(top, traffic=None) if top else None, "roofline_by_shape": table, "fp32_fma_tflops_measured": fma}
    if not args.no_cpu_baseline:
        cb = run_cpu(args, 3, 1, stack=True)
        res["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    return res


# ---------------------------------------------------------------------------------------------
# channel sweep (configs[4] of BASELINE.json): one JSON line per shape, stencil and dtype
# ---------------------------------------------------------------------------------------------
SWEEP = [(1, 16), (16, 16), (32, 64), (64, 128), (128, 128)]


def run_sweep(args, emit):
    import copy
    peaks = load_peaks()
    for k in (3, 1):
        for dtype in ("f32", "bf16"):
            if k == 1 and dtype == "bf16":
                continue                                     # the 1x1x1 stencil has one (fp32) implementation
            for cin, cout in SWEEP:
                a = copy.copy(args)
                a.layer, a.dtype = "%d,%d,0,%d" % (cin, cout, k), dtype
                a.steps, a.warmup = max(1, min(args.steps, 5)), max(3, min(args.warmup, 3))
                emit(run_layer(a, peaks))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the contract is ONE JSON line on
    # stdout, so everything else goes to stderr and the result is written to the saved descriptor at the end.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(result_fd, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        if rank != 0:
            return
        cb = run_cpu(args, max(1, args.steps), max(0, args.warmup))
        out = {"impl": "reference", "metric": "APR U-Net fwd+bwd particles/s", "value": cb["value"], "unit": "particles/s",
               "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"],
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
               "config": {"workload": "4-level APR U-Net fwd+bwd+SGD, reference CPU operators on host cores, bounded sample: " + cb["sample"]},
               "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
               "e2e": {"value": cb["value"], "unit": "particles/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit(out)
        return
    if args.config == 5 and not args.layer:
        run_sweep(args, emit)
        return
    if args.config == 4 and not args.batch_inference:
        args.batch_inference = 64
    if args.layer:
        out = run_layer(args)
    elif args.config == 2:
        out = run_block_stack(args)
    elif args.batch_inference:
        out = run_batch_inference(args)
    else:
        out = run_gpu(args)
    if out is not None:
        emit(out)


if __name__ == "__main__":
    main()
