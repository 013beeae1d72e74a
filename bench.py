"""Benchmark of the LUT-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  Rank 0 prints ONE
JSON line.  `value` is whole-job throughput with inputs resident in HBM; `e2e` is the same metric
through the public layer API with pinned-host inputs copied in and the result copied out inside the
timed region.  `roofline` describes the dominant kernel (algorithmic bytes / CUDA-event time against
the measured HBM peak), `cpu_baseline` the CPU oracle (a port of the reference's CPU path) timed on
a bounded sample on this host.  With --impl reference the CPU implementation itself is the arm.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML from a thread.  NVML is initialised in start() (before
    the warm-up), samples carry a host timestamp, and summary(t0, t1) reports those taken inside a timed region."""

    REASONS = {  # nvmlClocksEventReason* bit masks
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
    }

    def __init__(self, gpu_index, period_s=0.005):
        import threading
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []   # (time.perf_counter(), SM MHz, reason mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._error = None
        self._handle = None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML enumerates physical devices: honour CUDA_VISIBLE_DEVICES when it is a plain index list
            index = self.gpu_index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ids = [v.strip() for v in vis.split(",")]
                if index < len(ids) and ids[index].isdigit():
                    index = int(ids[index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception as e:  # NVML missing or restricted: report it instead of failing the run
            self._error = repr(e)
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        try:
            while not self._stop.is_set():
                mhz = float(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM))
                mask = self._nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                self.samples.append((time.perf_counter(), mhz, mask))
                time.sleep(self.period_s)
        except Exception as e:
            self._error = repr(e)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def summary(self, t0, t1, ms_per_step=None):
        inside = [(m, r) for (t, m, r) in self.samples if t0 <= t <= t1]
        reasons = set()
        for _, mask in inside:
            for bit, name in self.REASONS.items():
                if mask & bit:
                    reasons.add(name)
        med = statistics.median(m for m, _ in inside) if inside else None
        out = {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "samples": len(inside), "reasons": sorted(reasons),
               "window_s": t1 - t0}
        if med and ms_per_step:
            out["ms_per_step_x_mhz"] = ms_per_step * med   # clock-normalised step time (lower clock, longer step)
        if self._error:
            out["error"] = self._error
        return out


# ------------------------------------------------------------------------------------ workloads
class LutLayerWorkload:
    """Single fully connected LUT layer, forward + backward (train mode), fp32.

    Layer of the single-layer configuration: 784 inputs, 64 tables x 6 anchor pairs (64 rows), 32
    outputs; x uniform [0,1), tables N(0, 0.02), upstream gradient N(0,1).  The batch is raised above
    the configuration's 256 so that one step's inputs exceed L2 (the HBM roofline is meaningless on a
    12 MB step that is launch-latency bound).
    """

    metric = "LUT fwd+bwd samples/sec"
    unit = "samples/s"
    dtype = "f32"

    def l2_policy(self):
        """How cold caches are ensured between timed steps: the step's inputs exceed L2, or L2 is flushed."""
        return "inputs>L2" if getattr(self, "static_input_bytes", 0) > L2_BYTES else "flushed"

    def __init__(self, batch=65536, n_inputs=784, n_detectors=64, n_anchors=6, n_outputs=32, graph=False):
        self.B, self.I, self.Nt, self.Nc, self.O = batch, n_inputs, n_detectors, n_anchors, n_outputs
        self.name = f"single LUT layer fwd+bwd fp32 (I={n_inputs}, Nt={n_detectors}, Nc={n_anchors}, O={n_outputs}), batch {batch}"
        self.units_per_step = batch
        self.static_input_bytes = batch * (n_inputs + n_outputs) * 4
        # graph: the device-resident step (autograd forward + backward, 4 kernels of this library plus torch's
        # fills) is captured once into a CUDA graph and replayed; small batches are launch-latency bound otherwise
        self.graph = graph
        if graph:
            self.name += ", CUDA graph replay"

    def host_inputs(self, seed, batch):
        import synth
        x = synth.uniform(seed + 1, (batch, self.I))
        dY = synth.normal(seed + 2, (batch, self.O))
        return x, dY

    def structure(self):
        import synth
        anchors = synth.anchor_pairs(12, self.Nt, self.Nc, self.I)
        W = synth.normal(13, (self.Nt * (1 << self.Nc) * self.O,), 0.0, 0.02)
        return anchors, W

    def setup(self, device, rank):
        import torch
        from spiky_b200.lut_layer import LUTLayer, SynapseMeta

        anchors, W = self.structure()
        self.layer = LUTLayer(self.I, self.Nc, self.Nt, self.O, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                              _explicit_anchors=torch.from_numpy(anchors.reshape(-1)), device=device)
        with torch.no_grad():
            self.layer._weights.copy_(torch.from_numpy(W))
        self.layer.train()
        x, dY = self.host_inputs(1000 + rank, self.B)
        self.hx = torch.from_numpy(x).view(self.B, 1, self.I).pin_memory()
        self.hdy = torch.from_numpy(dY).view(self.B, 1, self.O).pin_memory()
        self.dx = self.hx.to(device)
        self.ddy = self.hdy.to(device)
        self.device = device
        self.h2d_bytes = self.hx.numel() * 4 + self.hdy.numel() * 4
        self.d2h_bytes = 4
        self.input_bytes = self.h2d_bytes
        self.cuda_graph = None
        if self.graph:
            from spiky_b200 import _native
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    self._run(self.dx, self.ddy)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            _native.profiler_reset()
            self.cuda_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.cuda_graph):
                self.graph_out = self._run(self.dx, self.ddy)
            self.graph_launches = sum(v["launches"] for v in _native.profiler_read().values())

    def _run(self, x, dy):
        x = x.detach().requires_grad_(True)
        self.layer._weights.grad = None
        y = self.layer(x)
        y.backward(dy)
        if self.allreduce is not None:
            self.allreduce([self.layer._weights])
        return y

    allreduce = None

    def trainable_parameters(self):
        return [self.layer._weights]

    def step_device(self):
        if self.cuda_graph is not None:
            self.cuda_graph.replay()
            return self.graph_out
        return self._run(self.dx, self.ddy)

    def step_e2e(self):
        """Host inputs -> device, one step, returns the device scalar the caller reads back."""
        if self.cuda_graph is not None:
            # the graph reads its inputs from fixed device buffers: copy this step's host batch into them
            self.dx.copy_(self.hx, non_blocking=True)
            self.ddy.copy_(self.hdy, non_blocking=True)
            self.cuda_graph.replay()
            return self.graph_out.sum()
        x = self.hx.to(self.device, non_blocking=True)
        dy = self.hdy.to(self.device, non_blocking=True)
        return self._run(x, dy).sum()

    # dominant kernel: the table-gradient scatter (2 x 4 x Nt x O bytes of row read-modify-write per sample)
    dominant_kernel = "fc_weight_grad"

    def traffic_key(self):
        # DRAM traffic was captured at batch 65536 only
        return "lut_layer_b65536" if self.B == 65536 and self.cuda_graph is None else None

    def algorithmic_bytes(self):
        """Per sample, by kernel family (every gathered / scattered row at full size, RMW counted twice)."""
        I, Nt, O = self.I, self.Nt, self.O
        return {
            "check_detectors": 4 * I + 12 * Nt,
            "fc_gather_forward": 4 * Nt + 4 * Nt * O + 4 * O,
            "fc_input_grad": 4 * O + 12 * Nt + 2 * 4 * Nt * O + 16 * Nt,
            "fc_weight_grad": 4 * O + 4 * Nt + 2 * 4 * Nt * O,
        }

    def cpu_step(self, batch, threads):
        """One forward+backward of `batch` samples on the CPU oracle; returns seconds."""
        from oracle import lut_oracle as orc
        anchors, W = self.structure()
        x, dY = self.host_inputs(77, batch)
        orc.set_threads(threads)
        t0 = time.perf_counter()
        y, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, self.Nt, self.Nc, self.O)
        orc.nonseq_fc_backward(W, dY, anchors, idx, md, mk, self.I, self.Nc)
        return time.perf_counter() - t0


class _Syncs:
    """Several table-update objects behind one wait() / remove()."""

    def __init__(self, parts):
        self.parts = list(parts)
        self.world = self.parts[0].world

    def wait(self):
        for p in self.parts:
            p.wait()

    def remove(self):
        for p in self.parts:
            p.remove()

    def __getattr__(self, name):   # the sharded update's own attributes (exchange_only, _plans, _on_backward)
        return getattr(self.parts[0], name)

    def __setattr__(self, name, value):
        if name in ("parts", "world"):
            object.__setattr__(self, name, value)
        else:
            setattr(self.parts[0], name, value)


class SparseConvNetWorkload:
    """Sparse LUT conv-net training step on 28x28 single-channel images (forward + backward + SGD).

    Network: three stacked ProjectionLUTLayers (5x5 receptive fields on a stride-2 grid of positions,
    32 / 64 / 128 tables per position, 8 anchor pairs = 256-row tables, 4x4 projections:
    28x28 -> 24x24 -> 20x20 -> 16x16) and a fully connected LUT readout (256 -> 10, 64 tables x 8 pairs).
    Input: ~19 % of the pixels non-zero, uniform in [0.5, 1); labels uniform over 10 classes (seeded
    synthetic stand-in for the digit images the reference trains on).  Loss: cross-entropy; optimiser:
    plain SGD on dense table gradients.
    """

    metric = "LUT fwd+bwd samples/sec"
    unit = "samples/s"
    dtype = "f32"
    LAYERS = [  # (in_hw, out_hw, grid, tables per position)
        (28, 24, 12, 32),
        (24, 20, 10, 64),
        (20, 16, 8, 128),
    ]
    NC = 8
    READOUT = (256, 10, 64, 8)  # inputs, outputs, tables, anchor pairs
    LR = 0.01

    def l2_policy(self):
        """How cold caches are ensured between timed steps: the step's inputs exceed L2, or L2 is flushed."""
        return "inputs>L2" if getattr(self, "static_input_bytes", 0) > L2_BYTES else "flushed"

    def __init__(self, batch=512, internal=False, sharded=False, peer=False, graph=False):
        self.B = batch
        self.units_per_step = batch
        # sharded: data parallelism without dense gradient exchange for the three sparse layers: ranks all-gather
        # (table index, output gradient) pairs, update their share of the detectors in place for the whole batch
        # and all-gather the updated tables (spiky_b200.data_parallel.ShardedTableUpdate); the readout layer keeps
        # all-reduce + SGD
        self.sharded = sharded
        # peer: data parallelism with the gradient reduction, the SGD update and the distribution of the updated tables
        # in one kernel over peer memory (spiky_b200.data_parallel.PeerTableUpdate), for all four layers
        self.peer = peer
        # graph: after the warm-up the device-resident step (forward, loss, backward, update, exchange) is captured into
        # one CUDA graph and replayed: no host work per step.  Offered where the step makes no NCCL call (one GPU, or
        # the peer-memory strategies, whose barriers count their epochs on the device).
        self.graph = graph
        self.graph_ok_multi = bool(peer) or sharded == "peer"
        # every step reads all tables: at least 16 synapses per row, 2^Nc rows per table (the exact figure, 382 MB, is
        # set when the layers are built); far beyond L2, so steps run back to back without a flush
        self.static_input_bytes = sum(g * g * per for _, _, g, per in self.LAYERS) * (1 << self.NC) * 16 * 4
        # internal: the reference's GradientType.Internal, the backward kernel applies W -= lr * dW in place (no dense
        # gradient, no optimiser pass); default: dense gradients + torch.optim.SGD
        self.internal = internal
        self.name = ("sparse LUT conv-net training step (3 ProjectionLUTLayers 32/64/128 tables per position, "
                     f"Nc=8, 5x5 receptive, stride 2, 4x4 projection + LUT readout to 10), batch {batch}"
                     + (", SGD update inside the backward kernel (Internal gradient policy)" if internal else ""))

    # ---- model
    def build(self, device):
        import torch
        import synth
        from spiky_b200.lut_layer import (GradientPolicy, GradientType, LUTLayer, ProjectionLUTLayer, SynapseMeta,
                                          PointSamplingPolicy, PointSamplingType)
        meta = SynapseMeta(min_weight=-1.0, max_weight=1.0)
        policy = GradientPolicy(GradientType.Internal if self.internal else GradientType.Dense)
        layers = []
        for li, (h, o, g, per) in enumerate(self.LAYERS):
            layer = ProjectionLUTLayer(
                (h, h), (o, o), self.NC, g * g, per, (5, 5), (4, 4), synapse_meta=meta,
                detectors_sampling_policy=PointSamplingPolicy(PointSamplingType.Grid, grid_h=g, grid_w=g, stride_h=2,
                                                              stride_w=2, pad_h=2, pad_w=2),
                weights_gradient_policy=policy, random_seed=100 + li)
            with torch.no_grad():
                layer._weights.normal_(0.0, 0.02, generator=torch.Generator().manual_seed(200 + li))
            layers.append(layer)
        I, O, Nt, Nc = self.READOUT
        readout = LUTLayer(I, Nc, Nt, O, synapse_meta=meta, weights_gradient_policy=policy, random_seed=104)
        with torch.no_grad():
            readout._weights.normal_(0.0, 0.02, generator=torch.Generator().manual_seed(204))
        layers.append(readout)
        if self.internal:
            for l in layers:
                l.set_external_learning_rate_hook(lambda w: self.LR)
        if device is not None:
            for l in layers:
                l.to(device=device)
        return layers

    def host_inputs(self, seed, batch):
        import synth
        x = synth.sparse_images(seed + 1, (batch, 28 * 28), density=0.19, lo=0.5, hi=1.0)
        labels = synth.integers(seed + 2, (batch,), 0, 10)
        return x, labels

    def setup(self, device, rank):
        import torch
        self.layers = self.build(device)
        for l in self.layers:
            l.train()
        params = [l._weights for l in self.layers]
        # every step reads all tables (382 MB): the step's inputs exceed L2, no flush between steps
        self.static_input_bytes = sum(p.numel() * p.element_size() for p in params)
        if self.sharded:
            from spiky_b200.data_parallel import ShardedTableUpdate
            self.table_sync = ShardedTableUpdate(self.layers[:-1], self.LR, batch_size=self.B,
                                                 transport="peer" if self.sharded == "peer" else "collectives",
                                                 share_copies=os.environ.get("BENCH_SHARE_COPIES", "stores"))
            # a replayed graph joins all its streams at its end: no overlap into the next step then
            self.overlaps_steps = self.sharded == "peer" and self.table_sync.world > 1 and not self.graph
            params = params[-1:]
            if self.sharded == "peer":
                # the small readout layer through the fused peer update: the step then has no NCCL call and no optimiser
                from spiky_b200.data_parallel import PeerTableUpdate
                self.table_sync = _Syncs([self.table_sync, PeerTableUpdate(self.layers[-1:], self.LR)])
                params = []
        if self.peer:
            from spiky_b200.data_parallel import PeerTableUpdate
            self.table_sync = PeerTableUpdate(self.layers, self.LR, barrier=os.environ.get("BENCH_PEER_BARRIER", "flags"))
            params = []
        self.opt = None if (self.internal or not params) else torch.optim.SGD(params, lr=self.LR)
        x, labels = self.host_inputs(1000 + rank, self.B)
        self.hx = torch.from_numpy(x).view(self.B, 1, 28, 28).pin_memory()
        self.hl = torch.from_numpy(labels).pin_memory()
        self.dx = self.hx.to(device)
        self.dl = self.hl.to(device)
        self.device = device
        self.h2d_bytes = self.hx.numel() * 4 + self.hl.numel() * 8
        self.d2h_bytes = 4
        self.grad_params = params

    cuda_graph = None
    graph_keeps_kernel_profile = True   # the per-kernel times of the line come from an eager pass of the same step

    def capture_graph(self):
        """Captures the device-resident step (inputs in self.dx / self.dl) into a CUDA graph."""
        import torch
        from spiky_b200 import _native
        if self.table_sync is not None:
            self.table_sync.wait()
        torch.cuda.synchronize()
        _native.profiler_reset()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.graph_out = self._run(self.dx, self.dl, join=True)
        self.graph_launches = sum(v["launches"] for v in _native.profiler_read().values())
        self.cuda_graph = g

    def _run(self, x, labels, join=False):
        import torch
        import torch.nn.functional as F
        if self.opt is not None:
            self.opt.zero_grad(set_to_none=True)
        if self.table_sync is not None and not self.overlaps_steps:
            self.table_sync.wait()  # the tables updated by the previous step have arrived
        z = x
        for l in self.layers[:-1]:
            z = l(z)
        logits = self.layers[-1](z.reshape(z.shape[0], 1, -1)).reshape(z.shape[0], -1)
        loss = F.cross_entropy(logits, labels)
        loss.backward()
        if self.internal:
            if self.average_tables is not None:
                self.average_tables()
        elif self.grad_sync is not None:
            # plain SGD, applied per table as soon as its gradient exchange has finished
            with torch.no_grad():
                for p in self.grad_sync.wait_each():
                    p.add_(p.grad, alpha=-self.LR)
        elif self.opt is not None:
            self.opt.step()
        if join and self.table_sync is not None:
            self.table_sync.wait()   # a captured step ends with every stream it used joined
        return loss

    allreduce = None
    grad_sync = None
    table_sync = None     # sharded / peer table update: the exchange it leaves running belongs to the step
    # True: every layer's forward pass waits for that layer's own exchange (the sharded update over peer memory), so the
    # exchange of the upper layers may run into the next step's forward pass of the lower ones; the timed region then
    # has no untimed gap between its steps and ends after the last exchange
    overlaps_steps = False
    average_tables = None  # data parallel + Internal policy: tables are averaged over the ranks after the step

    def trainable_parameters(self):
        return [] if self.internal else self.grad_params

    def step_device(self):
        if self.cuda_graph is not None:
            self.cuda_graph.replay()
            return self.graph_out
        return self._run(self.dx, self.dl)

    def step_e2e(self):
        if self.cuda_graph is not None:
            # The graph reads its inputs from fixed device buffers.  Every step's batch is copied from pinned host memory
            # into a staging pair on a copy stream while the previous step still runs, and moved into the graph's
            # buffers (device to device, microseconds) right before the replay: the host-to-device copy of step k + 1
            # overlaps step k instead of preceding its own step.
            import torch
            main = torch.cuda.current_stream(self.device)
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(device=self.device)
                self._sx, self._sl = torch.empty_like(self.dx), torch.empty_like(self.dl)
                self._staged, self._consumed = torch.cuda.Event(), torch.cuda.Event()
                self._prefetch(main)
            main.wait_event(self._staged)
            self.dx.copy_(self._sx, non_blocking=True)
            self.dl.copy_(self._sl, non_blocking=True)
            self._consumed.record(main)
            self.cuda_graph.replay()
            self._prefetch(None)   # the next step's batch
            return self.graph_out
        x = self.hx.to(self.device, non_blocking=True)
        labels = self.hl.to(self.device, non_blocking=True)
        return self._run(x, labels)

    _copy_stream = None

    def _prefetch(self, after):
        import torch
        with torch.cuda.stream(self._copy_stream):
            if after is not None:
                self._copy_stream.wait_stream(after)
            else:
                self._copy_stream.wait_event(self._consumed)   # the staging pair is free again
            self._sx.copy_(self.hx, non_blocking=True)
            self._sl.copy_(self.hl, non_blocking=True)
            self._staged.record(self._copy_stream)

    dominant_kernel = None  # picked by measured time

    def traffic_key(self):
        return "sparse_convnet_b512" if self.B == 512 else None

    def algorithmic_bytes(self):
        """Per sample and kernel family, summed over the layers that launch it."""
        out = {k: 0 for k in ("check_detectors", "sparse_forward", "sparse_input_grad", "sparse_weight_grad",
                              "fc_gather_forward", "fc_input_grad", "fc_weight_grad")}
        for li, (h, o, g, per) in enumerate(self.LAYERS):
            I, O, Nt = h * h, o * o, g * g * per
            sp = self._syn_per_sample.get((h, o), None)
            out["check_detectors"] += 4 * I + 12 * Nt
            out["sparse_forward"] += 4 * Nt + 4 * sp[0] + 4 * sp[1] + 4 * O
            if li > 0:  # the first layer's input is data: autograd asks for no input gradient, the pass is skipped
                out["sparse_input_grad"] += 4 * O + 12 * Nt + 2 * 4 * sp[0] + 16 * Nt
            out["sparse_weight_grad"] += 4 * O + 4 * Nt + 2 * 4 * sp[0]
        I, O, Nt, Nc = self.READOUT
        out["check_detectors"] += 4 * I + 12 * Nt
        out["fc_gather_forward"] += 4 * Nt + 4 * Nt * O + 4 * O
        out["fc_input_grad"] += 4 * O + 12 * Nt + 2 * 4 * Nt * O + 16 * Nt
        out["fc_weight_grad"] += 4 * O + 4 * Nt + 2 * 4 * Nt * O
        return out

    @property
    def _syn_per_sample(self):
        """(sum over detectors of synapses per row, sum over groups of targets) per projection layer."""
        res = {}
        for (h, o, g, per), l in zip(self.LAYERS, self.layers):
            sp = l._lut_dm._sparse
            res[(h, o)] = (sp.n_syn_per_sample, sp.n_syn_per_sample // per)
        return res

    # ---- CPU baseline: the same network and step on the CPU oracle
    def cpu_setup(self, fresh=False):
        """The network as numpy arrays for the oracle; cached (cpu_step trains it), fresh=True builds a new copy
        with the initial tables."""
        if fresh or getattr(self, "_cpu", None) is None:
            layers = self.build(None)
            cpu = []
            for l in layers[:-1]:
                idx = l._lut_dm._sparse
                cpu.append(dict(sp=dict(idx.numpy(), group_size=idx.group_size), W=l._weights.detach().numpy().copy(),
                                anchors=l._detector_anchors.numpy().copy(), I=l.n_inputs(), O=l.n_outputs()))
            r = layers[-1]
            cpu.append(dict(W=r._weights.detach().numpy().copy(), anchors=r._detector_anchors.numpy().copy()))
            if fresh:
                return cpu
            self._cpu = cpu
        return self._cpu

    def cpu_loss(self, x, labels):
        """Cross-entropy of the freshly built network on (x, labels), computed by the oracle."""
        import numpy as np
        from oracle import lut_oracle as orc
        cpu = self.cpu_setup(fresh=True)
        I, O, Nt, Nc = self.READOUT
        a = x
        for c in cpu[:-1]:
            a = orc.nonseq_sparse_forward(c["W"], a, c["anchors"], c["sp"], self.NC, c["O"])[0]
        logits = orc.nonseq_fc_forward(cpu[-1]["W"], a, cpu[-1]["anchors"], Nt, Nc, O)[0].astype(np.float64)
        z = logits - logits.max(axis=1, keepdims=True)
        logp = z - np.log(np.exp(z).sum(axis=1, keepdims=True))
        return float(-logp[np.arange(x.shape[0]), labels].mean())

    def parity_check(self, device):
        """The first step's loss on the GPU (freshly built network, the library's kernels, layers chained on the
        device) against the oracle's loss on the same batch."""
        import torch
        import torch.nn.functional as F
        layers = self.build(device)
        x, labels = self.host_inputs(77, self.B)
        with torch.no_grad():
            z = torch.from_numpy(x).view(self.B, 1, 28, 28).to(device)
            for l in layers[:-1]:
                l.train()
                z = l(z)
            layers[-1].train()
            logits = layers[-1](z.reshape(self.B, 1, -1)).reshape(self.B, -1)
            loss_gpu = float(F.cross_entropy(logits.double(), torch.from_numpy(labels).to(device)))
        loss_cpu = self.cpu_loss(x, labels)
        return {"loss_gpu": loss_gpu, "loss_oracle": loss_cpu, "rel": abs(loss_gpu - loss_cpu) / abs(loss_cpu),
                "what": f"cross-entropy of the first step's forward pass, batch {self.B}, same seeded batch and tables"}

    def cpu_step(self, batch, threads):
        import numpy as np
        from oracle import lut_oracle as orc
        cpu = self.cpu_setup()
        x, labels = self.host_inputs(77, batch)
        orc.set_threads(threads)
        I, O, Nt, Nc = self.READOUT
        t0 = time.perf_counter()
        acts, saved = [x], []
        for c in cpu[:-1]:
            y, idx, md, mk = orc.nonseq_sparse_forward(c["W"], acts[-1], c["anchors"], c["sp"], self.NC, c["O"])
            saved.append((idx, md, mk))
            acts.append(y)
        r = cpu[-1]
        logits, ridx, rmd, rmk = orc.nonseq_fc_forward(r["W"], acts[-1], r["anchors"], Nt, Nc, O)
        z = logits - logits.max(axis=1, keepdims=True)
        p = np.exp(z)
        p /= p.sum(axis=1, keepdims=True)
        p[np.arange(batch), labels] -= 1.0
        g = (p / batch).astype(np.float32)
        g, dW = orc.nonseq_fc_backward(r["W"], g, r["anchors"], ridx, rmd, rmk, I, Nc)
        r["W"] -= self.LR * dW
        for c, a, (idx, md, mk) in zip(reversed(cpu[:-1]), reversed(acts[:-1]), reversed(saved)):
            g, dW = orc.nonseq_sparse_backward(c["W"], g, c["anchors"], idx, md, mk, c["sp"], c["I"], self.NC)
            c["W"] -= self.LR * dW
        return time.perf_counter() - t0


class CharTransformerWorkload:
    """Character-level LUTTransformer training step (forward + cross-entropy + backward).

    vocab 65, context 128, batch 64, d_model 256, 4 layers, 4 heads, LUT attention (product mode, 2^8-row
    tables, 16 detectors per head, 4 positional dims) and LUT FFN / unembedder (16 detectors x 8 pairs), fp32
    tables N(0, 0.02).  Tokens are drawn from a Zipf(s=1.1) distribution over the 65 symbols (seeded synthetic
    stand-in for the byte-level text the reference trains on).  The configuration does not fix the number
    of detectors, the positional dimension or the attention mode; the values are the reference notebook's
    defaults, and product mode is the only one whose table size (2^Nc rows) matches the configuration.
    """

    metric = "LUTTransformer tokens/sec"
    unit = "tokens/s"
    dtype = "f32"
    dominant_kernel = None
    zipf_s = 1.1

    def traffic_key(self):
        return "char_transformer_b64" if (self.B, self.S, self.E, self.L) == (64, 128, 256, 4) else None

    def l2_policy(self):
        """How cold caches are ensured between timed steps: the step's inputs exceed L2, or L2 is flushed."""
        return "inputs>L2" if getattr(self, "static_input_bytes", 0) > L2_BYTES else "flushed"

    def __init__(self, batch=64, context=128, vocab=65, d_model=256, layers=4, heads=4, n_detectors=16, nc=8, npe=4):
        self.B, self.S, self.V, self.E, self.L, self.H = batch, context, vocab, d_model, layers, heads
        self.Nd, self.Nc, self.Npe = n_detectors, nc, npe
        self.units_per_step = batch * context
        self.name = (f"LUTTransformer training step (vocab {vocab}, context {context}, batch {batch}, d_model {d_model}, "
                     f"{layers} layers, {heads} heads, {n_detectors} detectors/head, Nc={nc}, product attention, Npe={npe})")

    def build(self, device):
        import torch
        from spiky_b200.lut_transformer import LUTTransformer
        from spiky_b200.lut_layer import SynapseMeta
        model = LUTTransformer(self.V, self.E, self.S, self.Npe, self.L, self.H, self.Nd, self.Nc,
                               concatenation_product=False, seed=11, device=device,
                               synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0))
        gen = torch.Generator().manual_seed(12)
        with torch.no_grad():
            for layer in model._lut_layers():
                layer._weights.copy_(torch.empty(layer._weights.shape).normal_(0.0, 0.02, generator=gen))
        return model

    def host_tokens(self, seed, batch):
        import torch
        p = torch.arange(1, self.V + 1, dtype=torch.float64) ** -self.zipf_s
        gen = torch.Generator().manual_seed(seed)
        return torch.multinomial(p / p.sum(), batch * (self.S + 1), replacement=True, generator=gen).view(batch, self.S + 1)

    def setup(self, device, rank):
        self.model = self.build(device)
        self.model.train()
        self.params = [p for p in self.model.parameters() if p.requires_grad]
        self.htok = self.host_tokens(1000 + rank, self.B).pin_memory()
        self.dtok = self.htok.to(device)
        self.device = device
        self.h2d_bytes = self.htok.numel() * 8
        self.d2h_bytes = 4

    allreduce = None

    def trainable_parameters(self):
        return self.params

    def _run(self, tok):
        import torch.nn.functional as F
        for p in self.params:
            p.grad = None
        logits = self.model(tok[:, :-1])
        loss = F.cross_entropy(logits.reshape(-1, self.V), tok[:, 1:].reshape(-1))
        loss.backward()
        if self.allreduce is not None:
            self.allreduce(self.params)
        return loss

    def step_device(self):
        return self._run(self.dtok)

    def step_e2e(self):
        return self._run(self.htok.to(self.device, non_blocking=True))

    def algorithmic_bytes(self):
        """Per token and kernel family, summed over the layers (attention: per token = (S-1)/2 pairs on average)."""
        E, V, Nt, Na, O = self.E, self.V, self.Nd, self.Nd * self.H, self.E
        pairs = (self.S - 1) / 2.0
        fc = lambda o: dict(fwd=4 * Nt + 4 * Nt * o + 4 * o, dx=4 * o + 12 * Nt + 8 * Nt * o + 16 * Nt, dw=4 * o + 4 * Nt + 8 * Nt * o)
        ffn, un = fc(E), fc(V)
        return {
            "check_detectors": (self.L + 1) * (4 * E + 12 * Nt),
            "fc_gather_forward": self.L * ffn["fwd"] + un["fwd"],
            "fc_input_grad": self.L * ffn["dx"] + un["dx"],
            "fc_weight_grad": self.L * ffn["dw"] + un["dw"],
            "product_forward": self.L * (pairs * Na * 4 * O + 4 * E + 4 * O),
            "product_backward": self.L * (pairs * Na * 16 * O + 4 * O + 8 * E),
            # histogram variant of the backward pass: the same algorithmic bytes, split over its kernels
            # (row pairs read for the input gradient; gradient rows read-modify-written; routing per token)
            "product_hist": self.L * 4 * E,
            "product_row_dots": self.L * pairs * Na * 8 * O,
            "product_route": self.L * (4 * O + 8 * E),
            "product_hist_weight_grad": self.L * pairs * Na * 8 * O,
            "product_hist_forward": self.L * (pairs * Na * 4 * O + 4 * O),
        }

    def cpu_step(self, batch, threads):
        """Forward + backward of `batch` sequences with the oracle's layer functions (same model)."""
        import numpy as np
        from oracle import lut_oracle as orc
        if getattr(self, "_cpu_model", None) is None:
            self._cpu_model = self.build(None)
        m = self._cpu_model
        tok = self.host_tokens(77, batch).numpy()
        orc.set_threads(threads)
        S, E, V = self.S, self.E, self.V
        t0 = time.perf_counter()
        z = m.token_embedder.weight.detach().numpy()[tok[:, :-1]]
        tape = []
        for block in m.layers:
            a, f = block["attention_lut"], block["ffn"]
            Wa, Aa = a._weights.detach().numpy(), a._detector_anchors.numpy()
            pe = a._prepare_positional_embeddings().detach().numpy().reshape(S - 1, a._n_detectors, -1)
            tape.append(("att", z.copy(), Wa, Aa, pe, a))
            z = z + orc.product_forward(Wa, z, pe, Aa, a._n_detectors, self.Nc, E, self.Npe)
            Wf, Af = f._weights.detach().numpy(), f._detector_anchors.numpy()
            y, idx, md, mk = orc.nonseq_fc_forward(Wf, z.reshape(-1, E), Af, self.Nd, self.Nc, E)
            tape.append(("ffn", Wf, Af, idx, md, mk))
            z = z + y.reshape(z.shape)
        u = m.unembedder
        Wu, Au = u._weights.detach().numpy(), u._detector_anchors.numpy()
        logits, idx, md, mk = orc.nonseq_fc_forward(Wu, z.reshape(-1, E), Au, self.Nd, self.Nc, V)
        p = np.exp(logits - logits.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        p[np.arange(p.shape[0]), tok[:, 1:].reshape(-1)] -= 1.0
        dz, _ = orc.nonseq_fc_backward(Wu, (p / p.shape[0]).astype(np.float32), Au, idx, md, mk, E, self.Nc)
        dz = dz.reshape(z.shape)
        for rec in reversed(tape):
            if rec[0] == "ffn":
                _, Wf, Af, idx, md, mk = rec
                dx, _ = orc.nonseq_fc_backward(Wf, dz.reshape(-1, E), Af, idx, md, mk, E, self.Nc)
                dz = dz + dx.reshape(dz.shape)
            else:
                _, zin, Wa, Aa, pe, a = rec
                dx, _, _ = orc.product_backward(Wa, zin, pe, Aa, dz, a._n_detectors, self.Nc, self.Npe)
                dz = dz + dx
        return time.perf_counter() - t0


class AttentionLayerWorkload:
    """One product-mode attention LUT layer of the character transformer, forward + backward: context 128, 256 inputs
    and outputs, 64 detectors x 8 anchor pairs (256-row tables), 4 positional dims; x uniform [0,1), tables N(0, 0.02),
    upstream gradient N(0,1).  Small enough for full ncu captures of the product-mode kernels."""

    metric = "LUT attention layer fwd+bwd tokens/sec"
    unit = "tokens/s"
    dtype = "f32"
    dominant_kernel = None

    def l2_policy(self):
        """How cold caches are ensured between timed steps: the step's inputs exceed L2, or L2 is flushed."""
        return "inputs>L2" if getattr(self, "static_input_bytes", 0) > L2_BYTES else "flushed"

    def __init__(self, batch=8, context=128, d_model=256, n_detectors=64, nc=8, npe=4):
        self.B, self.S, self.E, self.Nt, self.Nc, self.Npe = batch, context, d_model, n_detectors, nc, npe
        self.units_per_step = batch * context
        self.name = (f"product-mode attention LUT layer fwd+bwd (context {context}, batch {batch}, E=O={d_model}, "
                     f"Nt={n_detectors}, Nc={nc}, Npe={npe})")

    def setup(self, device, rank):
        import torch
        from spiky_b200.lut_layer import LUTLayer, SynapseMeta
        self.layer = LUTLayer(self.E, self.Nc, self.Nt, self.E, sequence_length=self.S,
                              synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0), concatenation_product=False,
                              positional_dim=self.Npe, random_seed=3, device=device)
        with torch.no_grad():
            self.layer._weights.copy_(torch.empty(self.layer._weights.shape).normal_(0.0, 0.02,
                                                                                     generator=torch.Generator().manual_seed(1)))
        self.layer.train()
        g = torch.Generator().manual_seed(1000 + rank)
        self.hx = torch.rand(self.B, self.S, self.E, generator=g).pin_memory()
        self.hdy = torch.randn(self.B, self.S, self.E, generator=g).pin_memory()
        self.dx, self.ddy = self.hx.to(device), self.hdy.to(device)
        self.device = device
        self.h2d_bytes = (self.hx.numel() + self.hdy.numel()) * 4
        self.d2h_bytes = 4

    allreduce = None

    def trainable_parameters(self):
        return [p for p in self.layer.parameters() if p.requires_grad]

    def _run(self, x, dy):
        for p in self.layer.parameters():
            p.grad = None
        x = x.detach().requires_grad_(True)
        y = self.layer(x)
        y.backward(dy)
        if self.allreduce is not None:
            self.allreduce(self.trainable_parameters())
        return y

    def step_device(self):
        return self._run(self.dx, self.ddy)

    def step_e2e(self):
        return self._run(self.hx.to(self.device, non_blocking=True), self.hdy.to(self.device, non_blocking=True)).sum()

    def algorithmic_bytes(self):
        E, Na = self.E, self.Nt
        pairs = (self.S - 1) / 2.0
        return {
            "product_forward": pairs * Na * 4 * E + 8 * E,
            "product_backward": pairs * Na * 16 * E + 12 * E,
            "product_hist": 4 * E,
            "product_row_dots": pairs * Na * 8 * E,
            "product_route": 12 * E,
            "product_hist_weight_grad": pairs * Na * 8 * E,
            "product_hist_forward": pairs * Na * 4 * E + 4 * E,
        }

    def cpu_step(self, batch, threads):
        import numpy as np
        from oracle import lut_oracle as orc
        orc.set_threads(threads)
        rng = np.random.default_rng(5)
        S, E, Na, Nc, Npe = self.S, self.E, self.Nt, self.Nc, self.Npe
        x = rng.random((batch, S, E), dtype=np.float32)
        dy = rng.standard_normal((batch, S, E)).astype(np.float32)
        a1 = rng.integers(0, 2 * E + Npe, (Na, Nc))
        anchors = np.stack([a1, (a1 + 1 + rng.integers(0, 2 * E + Npe - 1, (Na, Nc))) % (2 * E + Npe)], -1).astype(np.int32)
        W = (0.02 * rng.standard_normal((Na, 1 << Nc, E))).astype(np.float32)
        pe = rng.uniform(-1, 1, (S - 1, Na, Npe)).astype(np.float32)
        t0 = time.perf_counter()
        orc.product_forward(W, x, pe, anchors, Na, Nc, E, Npe)
        orc.product_backward(W, x, pe, anchors, dy, Na, Nc, Npe)
        return time.perf_counter() - t0


class LargeTransformerWorkload(CharTransformerWorkload):
    """Large LUTTransformer training step: vocab 32768 (Zipf s=1.05), context 1024, 32 sequences per GPU, d_model 1024,
    12 layers, 16 heads, 10 anchor pairs (1024-row tables), product attention with 16 detectors per head and 4
    positional dims.  One step is ~1e13 fp32 accumulations per layer, so the CPU sample runs one layer at context
    128 and extrapolates (attention cost by the number of causal pairs, per-token cost by the number of tokens)."""

    zipf_s = 1.05

    def __init__(self, batch=32):
        super().__init__(batch=batch, context=1024, vocab=32768, d_model=1024, layers=12, heads=16, n_detectors=16,
                         nc=10, npe=4)

    def cpu_step(self, batch, threads):
        import numpy as np
        from oracle import lut_oracle as orc
        orc.set_threads(threads)
        s, E, V, Nd, Na, Nc, Npe = 128, self.E, self.V, self.Nd, self.Nd * self.H, self.Nc, self.Npe
        rng = np.random.default_rng(5)
        x = rng.random((1, s, E), dtype=np.float32)
        dy = rng.standard_normal((1, s, E)).astype(np.float32)
        def anchors(nt, n_in):
            a1 = rng.integers(0, n_in, (nt, Nc))
            return np.stack([a1, (a1 + 1 + rng.integers(0, n_in - 1, (nt, Nc))) % n_in], -1).astype(np.int32)
        Wa = (0.02 * rng.standard_normal((Na, 1 << Nc, E))).astype(np.float32)
        Aa, pe = anchors(Na, 2 * E + Npe), rng.uniform(-1, 1, (s - 1, Na, Npe)).astype(np.float32)
        t0 = time.perf_counter()
        orc.product_forward(Wa, x, pe, Aa, Na, Nc, E, Npe)
        orc.product_backward(Wa, x, pe, Aa, dy, Na, Nc, Npe)
        t_att = time.perf_counter() - t0
        def per_token(o):
            W, A = (0.02 * rng.standard_normal((Nd, 1 << Nc, o))).astype(np.float32), anchors(Nd, E)
            g = rng.standard_normal((s, o)).astype(np.float32)
            t0 = time.perf_counter()
            _, idx, md, mk = orc.nonseq_fc_forward(W, x.reshape(s, E), A, Nd, Nc, o)
            orc.nonseq_fc_backward(W, g, A, idx, md, mk, E, Nc)
            return time.perf_counter() - t0
        t_ffn, t_un = per_token(E), per_token(V)
        S = self.S
        per_sequence = self.L * (t_att * (S * (S - 1)) / (s * (s - 1)) + t_ffn * S / s) + t_un * S / s
        self.cpu_note = (f"one attention layer, one FFN layer and the unembedder timed at context {s} on one sequence and "
                         f"extrapolated to {self.L} layers at context {S} (attention by causal pairs, the rest by tokens)")
        return per_sequence * batch


class LutInferWorkload:
    """Large single LUT layer, forward-only inference: 4096 inputs N(0,1), 4096 tables x 8 anchor pairs (256 rows)
    x 64 outputs; tables int8 uniform [-127,127] with one fp32 scale per table, or fp32 N(0, 0.02).  With N GPUs
    the tables (detectors) are sharded over the ranks, the batch is replicated, and one all-reduce combines
    the partial sums (int32 accumulators for int8 tables), so the job's throughput is that of the batch."""

    metric = "LUT forward samples/sec"
    unit = "samples/s"
    scaling = "strong"
    dominant_kernel = None

    def traffic_key(self):
        return "lut_infer_b16384" if self.B == 16384 and getattr(self, "world", 1) == 1 else None

    def l2_policy(self):
        """How cold caches are ensured between timed steps: the step's inputs exceed L2, or L2 is flushed."""
        return "inputs>L2" if getattr(self, "static_input_bytes", 0) > L2_BYTES else "flushed"

    def __init__(self, table_dtype="int8", batch=16384, n_inputs=4096, n_detectors=4096, n_anchors=8, n_outputs=64):
        self.kind = table_dtype
        self.dtype = "i8" if table_dtype == "int8" else "f32"
        self.B, self.I, self.Nt, self.Nc, self.O = batch, n_inputs, n_detectors, n_anchors, n_outputs
        self.units_per_step = batch
        self.static_input_bytes = batch * n_inputs * 4
        self.name = (f"single LUT layer inference, {table_dtype} tables (I={n_inputs}, Nt={n_detectors}, Nc={n_anchors}, "
                     f"O={n_outputs}), batch {batch}")

    def structure(self, n_detectors=None):
        import torch
        Nt = self.Nt
        gen = torch.Generator().manual_seed(5)
        a1 = torch.randint(0, self.I, (Nt, self.Nc), generator=gen)
        a2 = (a1 + torch.randint(1, self.I, (Nt, self.Nc), generator=gen)) % self.I
        anchors = torch.stack([a1, a2], dim=-1).to(torch.int32)
        n = Nt * (1 << self.Nc) * self.O
        if self.kind == "int8":
            tables = torch.randint(-127, 128, (n,), generator=gen, dtype=torch.int32).to(torch.int8)
            scales = (0.02 / 127) * (0.5 + torch.rand(Nt, generator=gen))
        else:
            tables = torch.empty(n).normal_(0.0, 0.02, generator=gen)
            scales = None
        return anchors, tables, scales

    def setup(self, device, rank):
        import torch
        import torch.distributed as dist
        from spiky_b200.inference import LUTInference
        world = dist.get_world_size() if dist.is_initialized() else 1
        anchors, tables, scales = self.structure()
        group = dist.group.WORLD if world > 1 else None
        self.layer = LUTInference.shard_of(rank if world > 1 else 0, world, self.I, self.O, self.Nt, self.Nc, anchors,
                                           tables, scales, int_rescaler=0.05, group=group, device=device)
        gen = torch.Generator().manual_seed(1000)   # the batch is replicated: same seed on every rank
        self.hx = torch.empty(self.B, self.I).normal_(generator=gen).pin_memory()
        self.dx = self.hx.to(device)
        self.device = device
        self.h2d_bytes = self.hx.numel() * 4
        self.d2h_bytes = 4
        self.world = world

    allreduce = None

    def trainable_parameters(self):
        return []

    def step_device(self):
        return self.layer(self.dx)

    def step_e2e(self):
        """The batch goes to the device in chunks on a copy stream while the previous chunk is computed."""
        import torch
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream()
        main = torch.cuda.current_stream()
        n_chunks = 4 if self.B >= 4096 else 1
        per = (self.B + n_chunks - 1) // n_chunks
        out = None
        self._copy_stream.wait_stream(main)   # device buffers of the previous step are free again
        for c in range(n_chunks):
            lo, hi = c * per, min(self.B, (c + 1) * per)
            with torch.cuda.stream(self._copy_stream):
                xc = self.hx[lo:hi].to(self.device, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record()
            main.wait_event(ready)
            xc.record_stream(main)
            y = self.layer(xc)
            out = y[0, 0] if out is None else out + y[0, 0]
        return out

    def algorithmic_bytes(self):
        e = 1 if self.kind == "int8" else 4
        Nt = self.Nt // getattr(self, "world", 1)
        gather = 4 * Nt + e * Nt * self.O + 4 * self.O + (4 * Nt if self.kind == "int8" else 0)
        return {"check_detectors": 4 * self.I + 4 * Nt, "int8_gather": gather, "fc_gather_forward": gather}

    def cpu_step(self, batch, threads):
        import numpy as np
        from oracle import lut_oracle as orc
        if getattr(self, "_cpu", None) is None:
            anchors, tables, scales = self.structure()
            if self.kind == "int8":
                W = (scales.numpy()[:, None] * tables.numpy().reshape(self.Nt, -1).astype(np.float32)).astype(np.float32)
            else:
                W = tables.numpy()
            self._cpu = (anchors.numpy(), W.reshape(-1))
        anchors, W = self._cpu
        x = np.random.default_rng(7).standard_normal((batch, self.I), dtype=np.float32)
        orc.set_threads(threads)
        t0 = time.perf_counter()
        orc.nonseq_fc_forward(W, x, anchors, self.Nt, self.Nc, self.O, train=False, int_mode=self.kind == "int8",
                              int_rescaler=0.05)
        return time.perf_counter() - t0


def _b(batch):
    """Keyword for the --batch override (None keeps the workload's configured batch)."""
    return {} if batch is None else {"batch": int(batch)}


WORKLOADS = {
    "lut_infer_int8": lambda batch=None: LutInferWorkload("int8", **_b(batch)),
    "lut_infer_fp32": lambda batch=None: LutInferWorkload("fp32", **_b(batch)),
    "char_transformer": lambda batch=None: CharTransformerWorkload(**_b(batch)),
    "attention_layer": lambda batch=None: AttentionLayerWorkload(**_b(batch)),
    "large_transformer": lambda batch=None: LargeTransformerWorkload(**_b(batch)),
    "large_transformer_b4": lambda batch=None: LargeTransformerWorkload(batch=batch or 4),
    "sparse_convnet": lambda batch=None: SparseConvNetWorkload(graph=True, **_b(batch)),
    "sparse_convnet_eager": lambda batch=None: SparseConvNetWorkload(**_b(batch)),
    "sparse_convnet_internal": lambda batch=None: SparseConvNetWorkload(internal=True, graph=True, **_b(batch)),
    "sparse_convnet_sharded": lambda batch=None: SparseConvNetWorkload(sharded=True, **_b(batch)),
    "sparse_convnet_sharded_peer": lambda batch=None: SparseConvNetWorkload(sharded="peer", **_b(batch)),
    "sparse_convnet_peer": lambda batch=None: SparseConvNetWorkload(peer=True, **_b(batch)),
    "sparse_convnet_peer_graph": lambda batch=None: SparseConvNetWorkload(peer=True, graph=True, **_b(batch)),
    "sparse_convnet_sharded_peer_graph": lambda batch=None: SparseConvNetWorkload(sharded="peer", graph=True, **_b(batch)),
    "lut_layer": lambda batch=None: LutLayerWorkload(**_b(batch)),
    "lut_layer_b256": lambda batch=None: LutLayerWorkload(batch=batch or 256),
    "lut_layer_b256_graph": lambda batch=None: LutLayerWorkload(batch=batch or 256, graph=True),
}
DEFAULT_WORKLOAD = "sparse_convnet"


def workload_config(wl):
    """The `config` object of the JSON line; both arms print exactly this for the same workload."""
    return {"workload": wl.name, "l2": wl.l2_policy(), "per_gpu_units": wl.units_per_step}


def _sample_sizes(wl):
    per_item = getattr(wl, "S", 1) if wl.unit == "tokens/s" else 1   # units per batch item
    return per_item, wl.units_per_step // per_item


def cpu_baseline(wl, budget_s=12.0):
    """Times the CPU oracle on a bounded sample of the workload (rank 0, N=1 only): all host threads (the figure
    reported), and one thread on a smaller sample (the reference's own CPU path is single-threaded)."""
    threads = os.cpu_count() or 1
    per_item, full = _sample_sizes(wl)
    batch = min(full, 256 if per_item == 1 else 1)
    dt = wl.cpu_step(batch, threads)  # warm-up and calibration
    per_unit = max(dt / batch, 1e-9)
    batch = int(max(batch, min(full, budget_s / 3 / per_unit)))
    times = [wl.cpu_step(batch, threads) for _ in range(3 if per_item == 1 else 1)]
    best = min(times)
    value = batch * per_item / best
    # one thread: a sample sized for ~3 s
    b1 = int(max(1, min(batch, 3.0 / (per_unit * threads))))
    t1 = wl.cpu_step(b1, 1)
    single = b1 * per_item / t1
    what = wl.unit.split("/")[0]
    if getattr(wl, "cpu_note", None):
        sample = wl.cpu_note + f", OpenMP ({threads} threads); one thread: {single:.4g} {wl.unit}"
    else:
        sample = (f"{batch} batch items ({batch * per_item} {what}) of the same workload, best of {len(times)}, OpenMP "
                  f"({threads} threads); one thread (the reference's own CPU path is single-threaded): {single:.4g} "
                  f"{wl.unit} on {b1} batch items")
    return {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample,
            "single_thread_value": single}


# ------------------------------------------------------------------------------------ arms
def run_reference(args):
    """The reference's CPU implementation of the path as the arm: the C oracle (a port pinned bit for bit to fixtures
    recorded from the reference's own CPU build) on all host threads, each step a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload](args.batch)
    threads = os.cpu_count() or 1
    per_item, full = _sample_sizes(wl)
    batch = min(full, 256 if per_item == 1 else 1)
    per_unit = max(wl.cpu_step(batch, threads) / batch, 1e-9)
    # each step is a bounded sample so that warmup + steps stay within ~2 minutes in total
    total = max(1, args.steps + args.warmup)
    batch = int(max(1 if per_item > 1 else 64, min(full, 100.0 / total / per_unit)))
    for _ in range(args.warmup):
        wl.cpu_step(batch, threads)
    times = [wl.cpu_step(batch, threads) for _ in range(args.steps)]
    ms = 1e3 * sum(times) / len(times)
    value = batch * per_item / (ms / 1e3)
    sample = (f"{batch} batch items ({batch * per_item} {wl.unit.split('/')[0]}) per step of the same workload, CPU oracle "
              f"(port of the reference CPU path), {threads} threads")
    if getattr(wl, "cpu_note", None):
        sample = f"{wl.cpu_note}; CPU oracle (port of the reference CPU path), {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": getattr(wl, "scaling", "weak"),
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": workload_config(wl),
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _attach_data_parallel(wl, world):
    """Gradient exchange of a data-parallel run: per-parameter all-reduce hooks (or the table average of the
    Internal policy); returns the sync object (None when there is nothing to exchange)."""
    import torch
    if world <= 1 or (not wl.trainable_parameters() and not getattr(wl, "internal", False)):
        return None
    # gradients are exchanged per parameter as soon as its backward has run, overlapping the rest of
    # the backward pass; the workload only waits for the outstanding collectives before it updates
    from spiky_b200.data_parallel import OverlappedGradientSync
    sync = OverlappedGradientSync(wl.trainable_parameters(), average=True)
    wl.allreduce = lambda params: sync.wait()
    wl.grad_sync = sync
    if getattr(wl, "internal", False):
        from spiky_b200.data_parallel import average_internal_policy_weights
        holder = torch.nn.ModuleList(wl.layers)
        wl.average_tables = lambda: average_internal_policy_weights(holder)
    return sync


def _dp_strategy(wl):
    tail = ", step replayed from a CUDA graph" if getattr(wl, "cuda_graph", None) is not None else ""
    if getattr(wl, "peer", False):
        return "fused update over peer memory" + tail
    if getattr(wl, "sharded", False) == "peer":
        return "sharded table update over peer memory" + tail
    return ("sharded table update" if getattr(wl, "sharded", False) else "gradient all-reduce") + tail


def _try_capture(wl, world, device):
    """Captures the workload's step into a CUDA graph when it asks for one; all ranks keep the graph or none does."""
    import torch
    import torch.distributed as dist
    if not getattr(wl, "graph", False) or getattr(wl, "cuda_graph", None) is not None:
        return
    if world > 1 and not getattr(wl, "graph_ok_multi", False):
        return   # the step makes NCCL calls from autograd hooks: issued eagerly
    ok = 1
    try:
        wl.capture_graph()
    except Exception as e:   # noqa: BLE001 - any failure means: run the step eagerly
        sys.stderr.write(f"graph capture failed, the step runs eagerly: {e}\n")
        ok = 0
    if world > 1:
        t = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = int(t)
    if not ok:
        wl.cuda_graph = None


def _replica_check(params, world):
    """max over parameters of the spread of a checksum over the ranks (0.0: the replicas hold identical tables)."""
    import torch
    import torch.distributed as dist
    if world <= 1 or not params:
        return None
    sums = torch.stack([torch.stack([p.detach().double().sum(), p.detach().abs().max().double()]) for p in params])
    lo, hi = sums.clone(), sums.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return float((hi - lo).abs().max())


def run_ours(args):
    import torch
    import torch.distributed as dist
    from spiky_b200 import _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback exists)"
    torch.cuda.set_device(local_rank)
    device = torch.device(f"cuda:{local_rank}")
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()   # NVML is up and sampling before the warm-up
    wl = WORKLOADS[args.workload](args.batch)
    wl.setup(device, rank)
    sync = _attach_data_parallel(wl, world)
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)
    dp_strategy = None
    if world > 1:
        dp_strategy = _dp_strategy(wl)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def finish_step(w):
        # exchanges a workload leaves running on a side stream belong to the step that started them
        if getattr(w, "table_sync", None) is not None:
            w.table_sync.wait()

    def timed_region(w, steps, profile):
        """Returns (ms per step measured with CUDA events on the current stream, profiler records, host window)."""
        _native.profiler_reset()
        _native.profiler_enable(profile)
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        do_flush = w.l2_policy() == "flushed"
        barrier()
        t0 = time.perf_counter()
        assert not (do_flush and getattr(w, "overlaps_steps", False)), "steps that overlap need back-to-back brackets"
        for i in range(steps):
            if do_flush:
                flush.zero_()
            starts[i].record()
            w.step_device()
            if i == steps - 1 or not getattr(w, "overlaps_steps", False):
                finish_step(w)
            stops[i].record()
        barrier()
        t1 = time.perf_counter()
        ms = sum(a.elapsed_time(b) for a, b in zip(starts, stops)) / steps
        prof = _native.profiler_read()
        _native.profiler_enable(False)
        return ms, prof, (t0, t1)

    if args.profile_only:
        # bare loop for profilers: warm-up + steps of the device-resident step, nothing else
        for _ in range(args.warmup + args.steps):
            wl.step_device()
        torch.cuda.synchronize()
        return
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        wl.step_device()
        finish_step(wl)
    _try_capture(wl, world, device)
    if world > 1:
        dp_strategy = _dp_strategy(wl)
    dp_trial = None
    if world > 1 and args.workload == DEFAULT_WORKLOAD and args.dp == "auto":
        # Ways to keep the replicas' tables equal (same SGD step, spiky_b200/data_parallel.py): all-reduce the dense
        # table gradients and run the optimiser; gather (index, output gradient) pairs and update a share of the tables
        # in place (through NCCL all-gathers, or with plain stores into peer memory); or reduce the dense gradients,
        # update and distribute in one kernel over peer memory.  Which one is fastest
        # depends on the number of ranks and on the interconnect: each is timed for a few steps and the fastest one
        # runs the measurement.
        def agreed(ms):
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        def release(w, s_):
            if s_ is not None:
                s_.remove()
            if getattr(w, "table_sync", None) is not None:
                w.table_sync.remove()

        best = (agreed(timed_region(wl, 8, profile=False)[0]), wl, sync)
        dp_trial = {_dp_strategy(wl): best[0]}
        for name in ("sparse_convnet_sharded", "sparse_convnet_peer", "sparse_convnet_sharded_peer",
                     "sparse_convnet_peer_graph", "sparse_convnet_sharded_peer_graph"):
            alt = WORKLOADS[name](args.batch)
            try:
                alt.setup(device, rank)
            except RuntimeError as e:
                # the constructors agree over the ranks before they raise, so every rank lands here together
                dp_trial[_dp_strategy(alt)] = "unavailable: " + str(e)[:200]
                continue
            alt_sync = _attach_data_parallel(alt, world)
            for _ in range(5):
                alt.step_device()
                finish_step(alt)
            _try_capture(alt, world, device)
            if getattr(alt, "graph", False) and alt.cuda_graph is None:
                dp_trial[_dp_strategy(alt) + ", step replayed from a CUDA graph"] = "unavailable: capture failed"
                release(alt, alt_sync)
                del alt
                torch.cuda.empty_cache()
                continue
            t_alt = agreed(timed_region(alt, 8, profile=False)[0])
            dp_trial[_dp_strategy(alt)] = t_alt
            if t_alt < best[0]:
                release(best[1], best[2])
                best = (t_alt, alt, alt_sync)
            else:
                release(alt, alt_sync)
            del alt
            torch.cuda.empty_cache()
        _, wl, sync = best
        dp_strategy = _dp_strategy(wl)
    # The figure: K steps with nothing but the step on the device.  The per-kernel times for the roofline come from a
    # second pass of the same K steps with the library's profiler on (two CUDA events around every launch): kept apart
    # because the extra event calls cost host time, which a step with many small launches on several streams feels.
    ms_dev, _, window = timed_region(wl, args.steps, profile=False)
    graph = getattr(wl, "cuda_graph", None)
    if graph is not None and getattr(wl, "graph_keeps_kernel_profile", False):
        # replayed launches do not pass through the library's entry points: the kernel times come from the same step
        # issued eagerly
        wl.cuda_graph = None
        for _ in range(2):
            wl.step_device()
            finish_step(wl)
        ms_profiled, prof, _ = timed_region(wl, args.steps, profile=True)
        wl.cuda_graph = graph
    else:
        ms_profiled, prof, _ = timed_region(wl, args.steps, profile=True)

    def e2e_region(steps):
        """End to end: every step copies its inputs from pinned host memory, runs, and its result is read back on the
        host; the read of step k is taken while step k+1 runs (two result slots), so the device never waits for the
        host.  Returns ms per step over the whole span (idle gaps and L2 flushes included)."""
        slots = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        done = [torch.cuda.Event() for _ in range(2)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        seen = []
        do_flush = wl.l2_policy() == "flushed"
        barrier()
        start.record()
        for i in range(steps):
            if do_flush:
                flush.zero_()
            r = wl.step_e2e()
            if i == steps - 1 or not getattr(wl, "overlaps_steps", False):
                finish_step(wl)
            slots[i % 2].copy_(r.detach().reshape(1).float(), non_blocking=True)
            done[i % 2].record()
            if i >= 1:
                done[(i - 1) % 2].synchronize()
                seen.append(float(slots[(i - 1) % 2][0]))
        stop.record()
        done[(steps - 1) % 2].synchronize()
        seen.append(float(slots[(steps - 1) % 2][0]))
        barrier()
        assert len(seen) == steps and all(v == v for v in seen), "a step's result was not read back"
        return start.elapsed_time(stop) / steps

    e2e_region(2)
    ms_e2e = e2e_region(args.steps)

    # host time per step: a few steps issued without waiting for the device (the launch queue absorbs them); well below
    # ms_per_step means the device sets the pace, close to it means the step is bound by the host's launch rate
    torch.cuda.synchronize()
    h0 = time.perf_counter()
    for _ in range(8):
        wl.step_device()
    host_ms = (time.perf_counter() - h0) / 8 * 1e3
    finish_step(wl)
    torch.cuda.synchronize()

    # ---- data-parallel evidence: replicas identical (checked BEFORE the run without exchange below, which lets
    # them drift on purpose), what the exchange costs, how fast the same payload moves alone
    replica = _replica_check([p for l in getattr(wl, "layers", []) for p in [l._weights]] or wl.trainable_parameters(), world)
    comm = None
    if world > 1 and getattr(wl, "sharded", False):
        # payload of the sharded update: every rank receives the other ranks' (index, output gradient) pairs and
        # table shares; the weight all-gather of the same sizes is timed alone for comparison
        tables = [l._weights for l in wl.layers[:-1]]
        pairs = sum(l.n_detectors() + 4 * l.n_outputs() for l in wl.layers[:-1]) * wl.B
        payload = (world - 1) * pairs + sum(p.numel() * p.element_size() for p in tables) * (world - 1) // world
        iso = []
        if wl.sharded == "peer":
            # the same stores and barriers with the update itself skipped (tables unchanged)
            ts = wl.table_sync
            ts.exchange_only = True
            for rep in range(4):
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for l in reversed(wl.layers[:-1]):
                    ts._on_backward(l, *ts._plans[id(l)]["last"], wl.B)
                ts.wait()
                b.record()
                torch.cuda.synchronize()
                iso.append(a.elapsed_time(b))
            ts.exchange_only = False
        else:
            shares = [torch.zeros((p.numel() + world - 1) // world, device=device) for p in tables]
            outs = [torch.empty(world * s_.numel(), device=device) for s_ in shares]
            for rep in range(4):
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for s_, o_ in zip(shares, outs):
                    dist.all_gather_into_tensor(o_, s_)
                b.record()
                torch.cuda.synchronize()
                iso.append(a.elapsed_time(b))
            del shares, outs
        comm = {"ms_local": 0.0, "ms_isolated": min(iso[1:]), "payload": payload, "sharded": wl.sharded}
    elif world > 1 and getattr(wl, "peer", False):
        # the fused update: a rank fetches its slice of the other ranks' gradients ((G-1)/G of the tables come in) and
        # stores its updated slice into their tables (as much goes out), while the others do the same with it: per GPU
        # and direction 2 (G-1)/G of the table bytes cross the links, what a ring all-reduce moves.  Timed as the
        # step without exchange (every rank updates its own copy from its own gradient) and alone (learning rate 0:
        # the same loads and stores, tables unchanged)
        ts = wl.table_sync
        payload = 2 * sum(l._weights.numel() * 4 for l in wl.layers) * (world - 1) // world
        ms_local = None
        if getattr(wl, "cuda_graph", None) is None:   # (a replayed graph has the exchange baked in)
            ts.paused = True
            for _ in range(2):
                wl.step_device()
                finish_step(wl)
            ms_local, _, _ = timed_region(wl, max(3, args.steps // 4), profile=False)
            ts.paused = False
        lr0, ts.lr = ts.lr, 0.0
        iso = []
        for rep in range(4):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for l in reversed(wl.layers):
                ts.gradient_ready(l)
            ts.wait()
            b.record()
            torch.cuda.synchronize()
            iso.append(a.elapsed_time(b))
        ts.lr = lr0
        comm = {"ms_local": ms_local, "ms_isolated": min(iso[1:]), "payload": payload, "peer": True}
    elif world > 1 and sync is not None and wl.trainable_parameters():
        params = wl.trainable_parameters()
        payload = sum(p.numel() * p.element_size() for p in params)
        sync.paused = True    # same step, gradients stay local: the difference is the exposed part of the exchange
        for _ in range(2):
            wl.step_device()
        ms_local, _, _ = timed_region(wl, max(3, args.steps // 4), profile=False)
        sync.paused = False
        bufs = [torch.zeros_like(p) for p in params]
        iso = []
        for rep in range(4):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for t in bufs:
                dist.all_reduce(t, op=dist.ReduceOp.AVG)
            b.record()
            torch.cuda.synchronize()
            iso.append(a.elapsed_time(b))
        del bufs
        comm = {"ms_local": ms_local, "ms_isolated": min(iso[1:]), "payload": payload}

    variants = None
    if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_secondary:
        # the same training step with the SGD update made inside the backward kernel (the reference's
        # GradientType.Internal): no dense gradient, no optimiser pass
        w1 = WORKLOADS["sparse_convnet_internal"](args.batch)
        w1.setup(device, rank)
        for _ in range(3):
            w1.step_device()
        _try_capture(w1, world, device)
        ms1, _, _ = timed_region(w1, 20, profile=False)
        variants = {"internal_gradient_policy": {"ms_per_step": ms1, "value": w1.units_per_step / (ms1 / 1e3),
                                                 "unit": w1.unit, "steps": 20}}
        del w1
        torch.cuda.empty_cache()
        # the default step with every launch issued by the host (the default replays the step from a CUDA graph)
        w1 = WORKLOADS["sparse_convnet_eager"](args.batch)
        w1.setup(device, rank)
        for _ in range(3):
            w1.step_device()
        ms1, _, _ = timed_region(w1, 20, profile=False)
        variants["launched_by_the_host"] = {"ms_per_step": ms1, "value": w1.units_per_step / (ms1 / 1e3), "unit": w1.unit,
                                            "steps": 20}
        del w1
        torch.cuda.empty_cache()
    secondary = None
    if args.workload == DEFAULT_WORKLOAD and not args.no_secondary:
        # the LUTTransformer half of the metric, measured in the same process on the same GPUs
        if sync is not None:
            sync.remove()
        for prm in wl.trainable_parameters():
            prm.grad = None
        torch.cuda.empty_cache()
        w2 = WORKLOADS["char_transformer"](None)
        w2.setup(device, rank)
        sync2 = _attach_data_parallel(w2, world)
        for _ in range(3):
            w2.step_device()
        ms2, _, _ = timed_region(w2, 10, profile=False)
        secondary = {"ms": ms2, "replica_check": _replica_check(w2.trainable_parameters(), world), "wl": w2}

    t = torch.tensor([ms_dev, ms_e2e, (comm["ms_local"] or 0.0) if comm else 0.0, comm["ms_isolated"] if comm else 0.0,
                      secondary["ms"] if secondary else 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e, ms_local, ms_isolated, ms_secondary = t.tolist()
    wait_errors = _native.device_wait_errors()
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(window[0], window[1], ms_dev)
        peak, peak_kind = measured_peaks()
        units = wl.units_per_step * (1 if getattr(wl, "scaling", "weak") == "strong" else world)
        value = units / (ms_dev / 1e3)
        launches = sum(v["launches"] for v in prof.values())
        alg = wl.algorithmic_bytes()
        if getattr(wl, "cuda_graph", None) is not None and getattr(wl, "graph_keeps_kernel_profile", False):
            launches = wl.graph_launches * args.steps
        elif getattr(wl, "cuda_graph", None) is not None:
            # replayed launches never pass through the library's entry points: count what the capture recorded and
            # take the whole replayed step as one launch of all kernels for the roofline
            launches = wl.graph_launches * args.steps
            alg = {"graph_step": sum(alg.values())}
            prof = {"graph_step": {"ms": ms_dev * args.steps, "timed": args.steps, "launches": args.steps}}
            wl.dominant_kernel = "graph_step"
        dom = wl.dominant_kernel or max((k for k in prof if prof[k]["timed"] and k in alg), key=lambda k: prof[k]["ms"])
        per_kernel = {}
        for k, v in prof.items():
            if v["timed"]:
                per_kernel[k] = {"ms_per_step": v["ms"] / args.steps, "launches_per_step": v["launches"] / args.steps,
                                 "alg_gbs": (alg.get(k, 0) * wl.units_per_step / 1e9) / (v["ms"] / args.steps / 1e3) if v["ms"] > 0 else None}
        # the family's launches of one step together move alg[dom] bytes per sample
        d = prof[dom]
        dom_ms = d["ms"] / max(d["timed"], 1)
        dom_ms_per_step = d["ms"] / args.steps
        achieved = alg[dom] * wl.units_per_step / 1e9 / (dom_ms_per_step / 1e3)
        traffic, traffic_note = ncu_traffic(wl, dom)
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_dev, "higher_is_better": True,
            "scaling": getattr(wl, "scaling", "weak"),
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": workload_config(wl),
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "traffic": (traffic / max(d["timed"] / args.steps, 1)) if traffic else None,
                         "traffic_source": traffic_note,
                         "algorithmic_bytes_per_launch": alg[dom] * wl.units_per_step / max(d["timed"] / args.steps, 1),
                         "ms_per_launch": dom_ms, "launches_per_step": d["timed"] / args.steps},
            "kernels": per_kernel,
            "e2e": {"value": units / (ms_e2e / 1e3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes, "ms_per_step": ms_e2e},
            "gpu_launches": int(launches),
            "host_ms_per_step": host_ms,
            "step_launch": "one CUDA graph replay per step" if getattr(wl, "cuda_graph", None) is not None
                           else "every kernel launched by the host",
            "ms_per_step_with_kernel_events": ms_profiled,
            "device_wait_errors": int(wait_errors),
            "clocks": clocks,
        }
        if comm and comm.get("sharded") == "peer":
            gb = comm["payload"] / 1e9
            line["comm"] = {
                "exchange": "every rank stores its (table index, output gradient) pairs into every rank's arrays, updates "
                            "its share of the tables in place for the whole batch and stores the share into every rank's "
                            "tables: plain stores into peer memory (CUDA IPC, NVLink), barriers through flags in peer "
                            "memory, overlapped with the backward pass",
                "payload_bytes_per_step_per_direction": comm["payload"], "isolated_ms": ms_isolated,
                "isolated_gbs_per_direction": gb / (ms_isolated / 1e3),
                "frac_of_nvlink": gb / (ms_isolated / 1e3) / 900.0,
                "frac_of_measured_peer_copy": gb / (ms_isolated / 1e3) / 770.0,
                "isolated_what": "the stores and barriers of one step alone, update skipped",
            }
        elif comm and comm.get("sharded"):
            gb = comm["payload"] / 1e9
            line["comm"] = {
                "exchange": "all-gather of (table index, output gradient) pairs, in-place update of a share of the tables, "
                            "all-gather of the updated shares (NCCL), overlapped with the backward pass",
                "payload_bytes_per_step": comm["payload"], "isolated_ms": ms_isolated,
                "isolated_busbw_gbs": gb / (ms_isolated / 1e3), "frac_of_nvlink": gb / (ms_isolated / 1e3) / 900.0,
                "isolated_what": "all-gather of the table shares alone (received bytes per rank / time)",
            }
        elif comm and comm.get("peer"):
            gb = comm["payload"] / 1e9
            line["comm"] = {
                "exchange": "one kernel per layer over peer memory (CUDA IPC, NVLink): each rank fetches its slice of every "
                            "rank's table gradient (bulk copies into a shared-memory ring), applies the SGD step and "
                            "stores the new slice into every rank's tables; overlapped with the backward pass of the "
                            "layers below; barriers through flags in peer memory",
                "payload_bytes_per_step_per_direction": comm["payload"],
                "ms_step_without_exchange": ms_local if comm["ms_local"] is not None else None,
                "exposed_ms": ms_dev - ms_local if comm["ms_local"] is not None else None, "isolated_ms": ms_isolated,
                "isolated_gbs_per_direction": gb / (ms_isolated / 1e3),
                "frac_of_nvlink": gb / (ms_isolated / 1e3) / 900.0,
                "frac_of_measured_peer_copy": gb / (ms_isolated / 1e3) / 770.0,
                "hidden_frac": 1.0 - (ms_dev - ms_local) / ms_isolated if comm["ms_local"] is not None else None,
            }
        elif comm:
            ring = 2.0 * (world - 1) / world * comm["payload"] / 1e9
            exposed = max(ms_dev - ms_local, 1e-6)
            line["comm"] = {
                "exchange": "all-reduce (NCCL, averaged) of every table gradient, overlapped with the backward pass",
                "payload_bytes_per_step": comm["payload"], "ms_step_without_exchange": ms_local,
                "exposed_ms": ms_dev - ms_local, "busbw_gbs": ring / (exposed / 1e3),
                "isolated_ms": ms_isolated, "isolated_busbw_gbs": ring / (ms_isolated / 1e3),
                "frac_of_nvlink": ring / (ms_isolated / 1e3) / 900.0,
                "hidden_frac": 1.0 - (ms_dev - ms_local) / ms_isolated,
            }
        if dp_strategy:
            line["dp_strategy"] = dp_strategy
            if dp_trial:
                line["dp_trial_ms_per_step"] = dp_trial
        if replica is not None:
            line["replica_check"] = replica
        if secondary:
            w2 = secondary["wl"]
            line["secondary"] = {"metric": w2.metric, "unit": w2.unit, "workload": w2.name, "steps": 10, "warmup": 3,
                                 "ms_per_step": ms_secondary, "value": w2.units_per_step * world / (ms_secondary / 1e3),
                                 "scaling": "weak"}
            if secondary["replica_check"] is not None:
                line["secondary"]["replica_check"] = secondary["replica_check"]
        if variants:
            line["variants"] = variants
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl)
            if hasattr(wl, "parity_check"):
                line["parity_check"] = wl.parity_check(device)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def ncu_traffic(wl, kernel):
    """DRAM bytes per step of a kernel family from the ncu capture summarised under profiles/ (dram_traffic.txt, JSON),
    valid only while the kernel's source file is the one that was profiled (sha256 recorded with the figure)."""
    import hashlib
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    key = getattr(wl, "traffic_key", None)
    if key is None or not os.path.exists(path):
        return None, None
    with open(path) as f:
        table = json.load(f)
    rec = table.get(key() if callable(key) else key, {}).get(kernel)
    if not rec:
        return None, None
    src = os.path.join(ROOT, "spiky_b200", "csrc", rec["source"])
    with open(src, "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()
    if sha != rec["sha256"]:
        return None, f"stale: {rec['source']} changed since the capture in {rec['summary']}"
    return rec["dram_bytes_per_step"], rec["summary"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's per-GPU batch (batch sweeps; the default is the configuration's batch)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle timing (batch sweeps)")
    ap.add_argument("--dp", default="auto", choices=["auto", "keep"],
                    help="data-parallel runs of the default workload: auto = time the exchange strategies for a few "
                         "steps and measure the fastest one; keep = the workload as named")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the character-transformer measurement that the default workload appends")
    ap.add_argument("--profile-only", action="store_true",
                    help="run only warm-up + steps of the device-resident step and exit (for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
