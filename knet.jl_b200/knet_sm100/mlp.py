"""The multi-layer perceptron of Knet's tutorial trained the way `minimize`/`adam!` does
(one forward+backward, then `update!` on every parameter: src/train20/train.jl:22-36), with
the batch dimension sharded over GPUs for data-parallel runs.

Model form (README.md:55-62, tutorial/40.mlp.ipynb): h = dropout(relu.(w*h .+ b), p) for the
hidden layers, scores = w*h .+ b, loss = nll(scores, labels).  Matrix products are cuBLAS
(through torch.mm); everything else runs in libknet_sm100: fused bias+relu+dropout forward,
fused nll forward/backward, dropback+reluback fused with the bias-gradient row sums of the
layer below, and a single multi-tensor optimizer launch.  Parameters, gradients and optimizer state live
in flat buffers so that a layer's gradients are one contiguous all-reduce bucket.
"""
import ctypes as C

import numpy as np
import torch

from . import dp, ops
from .karray import KnetArray
from .lib import knet, knet8, libknet, ptr, sfx
from .train import Adam, Momentum, MultiTensorPlan, SGD, update_multi_


class MLP:
    def __init__(self, sizes, batch, pdrop=0.0, dtype=torch.float32, seed=1, optimizer=None,
                 device="cuda", process_group=None, weights=None, dropout_seed=None, shard_update=False,
                 fuse_bias_grad=True):
        """sizes = [in, hidden..., out]; `weights` optionally gives host (w, b) NumPy pairs
        (column-major Julia shapes) instead of the xavier draw; `process_group` turns on the
        gradient all-reduce (one rank per GPU, same weights everywhere, batch sharded).
        `shard_update` replaces it by reduce-scatter -> update of the rank's own 1/world of
        every layer -> all-gather of the weights, with optimizer state kept for that shard only.
        `fuse_bias_grad=False` computes the hidden layers' bias gradients with a separate
        sum(dz, dims=2) instead of inside the dropback+reluback kernel."""
        self.sizes, self.batch, self.pdrop, self.dtype = list(sizes), batch, pdrop, dtype
        self.device = torch.device(device)
        self.S = sfx(dtype)
        self.esize = 4 if dtype == torch.float32 else 8
        self.ct = C.c_float if dtype == torch.float32 else C.c_double
        self.opt = optimizer if optimizer is not None else Adam()
        self.pg = process_group
        if isinstance(process_group, dp.KnetComm):
            self.world = process_group.world
        else:
            self.world = torch.distributed.get_world_size(process_group) if process_group is not None else 1
        self.seed, self.step_no = (seed if dropout_seed is None else dropout_seed), 0
        L = len(sizes) - 1
        self.L = L
        counts = [sizes[i + 1] * sizes[i] + sizes[i + 1] for i in range(L)]
        if isinstance(process_group, dp.KnetComm):
            self.rank = process_group.rank
        else:
            self.rank = torch.distributed.get_rank(process_group) if process_group is not None else 0
        self.sharded = bool(shard_update) and self.world > 1
        if self.sharded:
            self.offsets = np.asarray(dp.padded_offsets(counts, self.world), dtype=np.int64)
        else:
            self.offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        total = int(self.offsets[-1])
        self.flat_w = torch.zeros(total, dtype=dtype, device=self.device)
        self.flat_g = torch.zeros(total, dtype=dtype, device=self.device)
        self.state = []
        nstate = total // self.world if self.sharded else total
        if isinstance(self.opt, (Adam, Momentum)):
            self.state.append(torch.zeros(nstate, dtype=dtype, device=self.device))
        if isinstance(self.opt, Adam):
            self.state.append(torch.zeros(nstate, dtype=dtype, device=self.device))
        self.gather_works = [None] * L
        rng = np.random.default_rng(seed)
        npdt = np.float32 if dtype == torch.float32 else np.float64
        self.w, self.b, self.dw, self.db = [], [], [], []
        arrays = []
        for i in range(L):
            o, n_in, n_out = int(self.offsets[i]), sizes[i], sizes[i + 1]
            nw = n_out * n_in
            if weights is not None:
                w_host, b_host = weights[i]
            else:
                u = rng.random((n_out, n_in))
                s = np.sqrt(6.0 / (n_in + n_out))
                w_host, b_host = ((2 * s) * u - s).astype(npdt), np.zeros(n_out, dtype=npdt)
            self.flat_w[o:o + nw].copy_(torch.from_numpy(
                np.ascontiguousarray(np.asfortranarray(w_host).reshape(-1, order="F").astype(npdt))))
            self.flat_w[o + nw:o + nw + n_out].copy_(torch.from_numpy(np.ascontiguousarray(b_host.astype(npdt))))
            self.w.append(KnetArray(self.flat_w[o:o + nw], (n_out, n_in)))
            self.b.append(KnetArray(self.flat_w[o + nw:o + nw + n_out], (n_out,)))
            self.dw.append(KnetArray(self.flat_g[o:o + nw], (n_out, n_in)))
            self.db.append(KnetArray(self.flat_g[o + nw:o + nw + n_out], (n_out,)))
            if self.sharded:      # one array per layer: this rank's slice of the padded bucket
                lo, hi = dp.shard_bounds((o, int(self.offsets[i + 1])), self.rank, self.world)
                so = o // self.world
                arrays.append((self.flat_w[lo:hi], self.flat_g[lo:hi]) +
                              tuple(s[so:so + hi - lo] for s in self.state))
                continue
            for (a, n) in ((o, nw), (o + nw, n_out)):
                arrays.append((self.flat_w[a:a + n], self.flat_g[a:a + n]) +
                              tuple(s[a:a + n] for s in self.state))
        self.plan = MultiTensorPlan(arrays)
        # sharded update: one plan per layer as well, so that a layer's weights can start their
        # all-gather as soon as that layer's shard is updated
        self.layer_plans = [MultiTensorPlan([a]) for a in arrays] if self.sharded else None
        # activations: h[i] is the output of layer i (after relu/dropout), reused as its own
        # gradient buffer on the way back
        self.h = [KnetArray.empty((sizes[i + 1], batch), dtype, self.device) for i in range(L)]
        self.dh = [KnetArray.empty((sizes[i + 1], batch), dtype, self.device) for i in range(L)]
        self.total = torch.zeros(1, dtype=dtype, device=self.device)
        self.count = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.per_instance = torch.empty(batch, dtype=dtype, device=self.device)
        self.launches = 0
        self.fuse_bias_grad = bool(fuse_bias_grad)
        # dropout counters: layer i of step t uses [t*per_step + base[i], ... + groups[i]), disjoint ranges
        groups = [ops.philox_groups(sizes[i + 1] * batch, dtype) for i in range(L - 1)]
        self._drop_base = [sum(groups[:i]) for i in range(L - 1)]
        self._drop_per_step = sum(groups)
        self.probe = None          # optional object with begin(label, bytes) / end(): times every library launch
        self._rs_works, self._pending = {}, []      # sharded update: reduce-scatters in flight, layers not yet updated
        self._graph, self._capturing = None, False
        if self.sharded and getattr(self.opt, "gclip", 0):
            # the plan holds one slice per layer and rank, so per-array norms (gclip!, update.jl:572-583)
            # would be taken over parts of arrays
            raise ValueError("gradient clipping is not available with shard_update")

    def _kn(self, label, nbytes, call, *args, launches=1):
        """One library call; `nbytes` is its algorithmic traffic (for the optional probe)."""
        if self.probe is not None:
            self.probe.begin(label, nbytes)
        call(*args)
        if self.probe is not None:
            self.probe.end()
        self.launches += launches

    # ---- pieces ---------------------------------------------------------------------------
    def params(self):
        out = []
        for w, b in zip(self.w, self.b):
            out += [w, b]
        return out

    def forward(self, x, uniforms=None, train=True):
        """x: KnetArray (in, batch).  `uniforms` (one KnetArray per hidden layer) selects the
        unfused path with supplied U[0,1) draws, as Knet's dropout!(p,x,y) consumes them."""
        h = x
        B = self.batch
        for i in range(self.L):
            z = self.h[i]
            if self.gather_works[i] is not None:      # this layer's updated weights have arrived
                self.gather_works[i].wait()
                self.gather_works[i] = None
            ops.matmul(self.w[i], h, out=z)
            n_out = self.sizes[i + 1]
            n = n_out * B
            es = self.esize
            if i < self.L - 1:
                p = self.pdrop if train else 0.0
                if uniforms is None and self._graph is not None and self._capturing:
                    # counter offset = the layer's base (fixed) + step_no*per_step (device memory, refreshed per replay)
                    self._kn("bias+relu+dropout fwd", (2 * n + n_out) * es, knet, f"knet_bias_relu_dropout_fwd_g_{self.S}",
                             ptr(z.data), ptr(self.b[i].data), ptr(z.data), n_out, B, self.ct(p), self.seed, self._drop_base[i],
                             C.c_void_p(self._dev_step.data_ptr() + 8 * i))
                elif uniforms is None:
                    off = self.step_no * self._drop_per_step + self._drop_base[i]
                    self._kn("bias+relu+dropout fwd", (2 * n + n_out) * es, knet, f"knet_bias_relu_dropout_fwd_{self.S}",
                             ptr(z.data), ptr(self.b[i].data), ptr(z.data), n_out, B, self.ct(p), self.seed, off)
                else:
                    knet8(f"add_{self.S}_12", n, ptr(z.data), 1, n, ptr(self.b[i].data), 1, n_out, ptr(z.data))
                    knet8(f"relu_{self.S}", n, ptr(z.data), ptr(z.data))
                    self.launches += 2
                    if p > 0:
                        u = uniforms[i].data.clone()
                        knet8(f"dropout_{self.S}", n, self.ct(p), ptr(z.data), ptr(u))
                        z.data.copy_(u)
                        self.launches += 1
            else:
                self._kn("bias add (output layer)", (2 * n + n_out) * es, knet8, f"add_{self.S}_12", n, ptr(z.data), 1, n,
                         ptr(self.b[i].data), 1, n_out, ptr(z.data))
            h = z
        return h

    def loss(self, scores, labels):
        n = self.sizes[-1] * self.batch
        self._kn("nll fwd", n * self.esize + 4 * self.batch, knet, f"knet_nll_fwd_{self.S}", ptr(scores.data), ptr(labels),
                 self.sizes[-1], self.batch, 1, ptr(self.total), ptr(self.count), ptr(self.per_instance), launches=2)
        return self.total, self.count

    def backward(self, x, labels):
        """Gradients of the mean loss into flat_g; per-layer all-reduce buckets are issued as
        soon as a layer's dW and db are final, overlapping the rest of the backward pass."""
        B = self.batch
        works = []
        self._rs_works, self._pending = {}, list(range(self.L)) if self.sharded else []
        scores = self.h[-1]
        dz = self.dh[-1]
        es = self.esize
        self._kn("nll bwd", 2 * self.sizes[-1] * B * es + 4 * B, knet, f"knet_nll_bwd_{self.S}", ptr(scores.data),
                 ptr(labels), self.sizes[-1], B, 1, 1, self.ct(1.0), ptr(self.count), ptr(dz.data))
        for i in reversed(range(self.L)):
            n_out = self.sizes[i + 1]
            hin = x if i == 0 else self.h[i - 1]
            # db = sum(dz, dims=2) (the hidden layers' came with their dz); dW = dz * hin'
            if i == self.L - 1 or not self.fuse_bias_grad:
                self._kn("bias gradient sum dims=2", (n_out * B + n_out) * es, knet8, f"sum_{self.S}_21", n_out * B,
                         ptr(dz.data), 1, n_out, ptr(self.db[i].data))
            ops.A_mul_Bt(dz, hin, out=self.dw[i])
            if self.sharded:
                self._rs_works[i] = dp.reduce_scatter_bucket(self.flat_g, (int(self.offsets[i]), int(self.offsets[i + 1])),
                                                             self.rank, self.world, group=self.pg)
                if i + 1 < self.L:      # the layer above was reduced under this layer's products: update it now
                    self._update_layer(i + 1)
            elif self.pg is not None and self.world > 1:
                works.append(dp.allreduce_bucket(self.flat_g, (int(self.offsets[i]), int(self.offsets[i + 1])),
                                                 group=self.pg))
            if i > 0:
                dprev = self.dh[i - 1]
                ops.At_mul_B(self.w[i], dz, out=dprev)
                n = self.sizes[i] * B
                if self.fuse_bias_grad:
                    self._kn("dropback+reluback+bias gradient bwd", (3 * n + self.sizes[i]) * es, knet,
                             f"knet_relu_dropout_bias_bwd_{self.S}", ptr(hin.data), ptr(dprev.data), ptr(dprev.data),
                             ptr(self.db[i - 1].data), self.sizes[i], B, self.ct(self.pdrop))
                else:
                    self._kn("dropback+reluback bwd", 3 * n * es, knet, f"knet_relu_dropout_bwd_{self.S}", ptr(hin.data),
                             ptr(dprev.data), ptr(dprev.data), n, self.ct(self.pdrop))
                dz = dprev
        for w in works:
            w.wait()

    def update(self):
        nupd = int(self.offsets[-1]) // self.world if self.sharded else int(self.offsets[-1])
        per_param = (3 + 2 * len(self.state)) * self.esize          # read w, g, state; write w, state
        if self._capturing and isinstance(self.opt, Adam):
            self._kn("update! (multi-tensor)", nupd * per_param, knet, f"knet_adam_multi_g_{self.S}", ptr(self.plan.table),
                     self.plan.ntensors, self.plan.total_chunks, self.opt.lr, self.opt.beta1, self.opt.beta2, self.opt.eps,
                     C.c_void_p(self._dev_step.data_ptr() + 8 * self.L), dp.gradient_scale(self.world))
        elif self.sharded:
            for i in sorted(self._pending):       # what backward() has not updated yet (the first layer)
                self._update_layer(i)
        else:
            self._kn("update! (multi-tensor)", nupd * per_param, update_multi_, self.plan, self.opt,
                     dp.gradient_scale(self.world))

    def _update_layer(self, i):
        """Sharded update of one layer: wait for its reduce-scatter, update this rank's shard (one
        launch), start the all-gather of the layer's weights on the side stream.  backward() calls
        it for layer i+1 once layer i's products are queued, so everything but the first layer's
        exchange runs under the remaining backward products; Adam's step count advances with the
        first layer updated in a step."""
        self._rs_works.pop(i).wait()
        n_i = (int(self.offsets[i + 1]) - int(self.offsets[i])) // self.world
        per_param = (3 + 2 * len(self.state)) * self.esize
        self._kn("update! (own shard of one layer)", n_i * per_param, update_multi_, self.layer_plans[i], self.opt,
                 dp.gradient_scale(self.world), len(self._pending) == self.L)
        self._pending.remove(i)
        self.gather_works[i] = dp.allgather_bucket(
            self.flat_w, (int(self.offsets[i]), int(self.offsets[i + 1])), self.rank, self.world, group=self.pg)

    def sync_weights(self):
        """Wait for the weight all-gathers of a sharded update (before reading flat_w)."""
        for i, w in enumerate(self.gather_works):
            if w is not None:
                w.wait()
                self.gather_works[i] = None

    def step(self, x, labels, uniforms=None):
        """One training step; returns the device scalars (total, count) of the local loss."""
        scores = self.forward(x, uniforms)
        self.loss(scores, labels)
        self.backward(x, labels)
        self.update()
        self.step_no += 1
        return self.total, self.count

    # ---- the whole step as one CUDA graph (launch-bound sizes) -------------------------------------
    # Everything that changes from step to step and is passed by value in the eager step - the
    # dropout counter offsets and Adam's bias corrections - is read from a small device buffer
    # instead, which one host-to-device copy refreshes before each replay; the scalars are
    # computed on the host exactly as the eager entry points compute them, so a replayed step
    # is bit-identical to an eager one.
    _SLOTS = 32

    def capture(self):
        """Record forward + loss + backward + update into a CUDA graph (single GPU).  Afterwards
        `step_graph(x, labels)` runs a step with one graph launch."""
        if self.world > 1:
            raise NotImplementedError("the captured step is for one GPU")
        L, esz = self.L, 4 if self.dtype == torch.float32 else 8
        nbytes = 8 * L + 2 * esz
        self._dev_step = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self._host_step = torch.zeros((self._SLOTS, nbytes), dtype=torch.uint8).pin_memory()
        self._slot_free = [None] * self._SLOTS
        self.gx = KnetArray.empty((self.sizes[0], self.batch), self.dtype, self.device)
        self.gy = torch.zeros(self.batch, dtype=torch.int32, device=self.device)
        self._graph = torch.cuda.CUDAGraph()
        saved = (self.flat_w.clone(), [s.clone() for s in self.state], self.step_no, getattr(self.opt, "t", 0),
                 self.launches)
        self.gx.data.normal_()
        self.gy.fill_(1)
        self._capturing = True
        try:
            self._refresh_step_scalars()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                  # warm-up off the capture: lazy initialisations
                for _ in range(2):
                    self._run_step_body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            l0 = self.launches
            with torch.cuda.graph(self._graph):
                self._run_step_body()
            self.launches_per_replay = self.launches - l0
        finally:
            self._capturing = False
        self.flat_w.copy_(saved[0])
        for s, c in zip(self.state, saved[1]):
            s.copy_(c)
        self.step_no, self.launches = saved[2], saved[4]
        if hasattr(self.opt, "t"):
            self.opt.t = saved[3]
        torch.cuda.synchronize()
        return self

    def _run_step_body(self):
        scores = self.forward(self.gx)
        self.loss(scores, self.gy)
        self.backward(self.gx, self.gy)
        self.update()

    def _refresh_step_scalars(self):
        """Host side of a replayed step: counter offsets of this step and Adam's bias corrections
        for t + 1 into a pinned slot, then one async copy to the device buffer the graph reads."""
        import numpy as np
        L = self.L
        slot = self.step_no % self._SLOTS
        if self._slot_free[slot] is not None:
            self._slot_free[slot].synchronize()           # its previous copy has left the host buffer
        row = self._host_step[slot].numpy()
        offs = row[:8 * L].view(np.uint64)
        for i in range(L - 1):
            offs[i] = self.step_no * self._drop_per_step
        if isinstance(self.opt, Adam):
            t = self.opt.t + 1
            bc = row[8 * L:].view(np.float32 if self.dtype == torch.float32 else np.float64)
            getattr(libknet, f"knet_adam_bias_corr_{self.S}")(self.opt.beta1, self.opt.beta2, t,
                                                              C.c_void_p(bc.ctypes.data))
        self._dev_step.copy_(self._host_step[slot], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._slot_free[slot] = ev

    def step_graph(self, x=None, labels=None):
        """One training step through the captured graph.  x / labels are copied into the graph's
        input buffers unless they are those buffers (`self.gx`, `self.gy`) already."""
        if self._graph is None:
            raise RuntimeError("call capture() first")
        if x is not None and x is not self.gx:
            self.gx.data.copy_(x.data, non_blocking=True)
        if labels is not None and labels is not self.gy:
            self.gy.copy_(labels, non_blocking=True)
        self._refresh_step_scalars()
        self._graph.replay()
        if isinstance(self.opt, Adam):
            self.opt.t += 1
        self.step_no += 1
        self.launches += self.launches_per_replay
        return self.total, self.count
