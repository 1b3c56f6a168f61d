"""Host-side sequence of a batch-sharded (synchronised) training batch norm + activation chain.

One process per GPU; every rank holds a contiguous slab of the batch. The only communication is one
all-reduce of 2*C floats in the forward pass ({sum x, sum x^2}) and one in the backward pass
({sum du, sum du*xhat}); everything else is per-rank work. nnForge itself does not synchronise batch
statistics across devices (its multi-GPU path all-reduces weight gradients only,
nnforge/cuda/backward_propagation_cuda.cpp:963-971), so with one rank the result equals the reference's.

`kernels` is the compute backend: on a GPU `nnforge_b200.capi`; the CPU tests pass an adapter over the
checker so that this file's logic (buffer roles, what is reduced, which sums feed which call) runs under
`gloo` without a GPU. The per-channel weight gradients accumulate the LOCAL sums, as the reference
leaves their cross-device sum to its own gradient all-reduce.
"""
import torch
import torch.distributed as dist


def _world(group):
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


class NcclExchange:
    """In-place sum over ranks through torch.distributed (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        self.group = group

    def all_reduce(self, tensor):
        dist.all_reduce(tensor, group=self.group)


class PeerExchange:
    """In-place sum over the GPUs of one machine through peer memory (nnf_peer_* entry points): every rank
    stores its message into all ranks' symmetric buffers and sums what arrives in its own, which costs two
    ~2 us launches plus one NVLink store latency instead of an NCCL launch. The symmetric buffers come from
    torch.distributed._symmetric_memory; construction is collective."""

    def __init__(self, kernels, kmax, device, group=None):
        import os
        # plain peer loads/stores only: no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.k = kernels
        self.kmax = kmax
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        floats = kernels.peer_exchange_bytes(kmax) // 4
        self.buf = symm_mem.empty(floats, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.seq = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)  # every buffer is zeroed before anyone publishes into it

    def all_reduce(self, tensor):
        self.seq += 1
        self.k.peer_exchange_sum(tensor, tensor, self.ptrs, self.rank, self.world, self.kmax, self.seq)

    def next_seq(self):
        self.seq += 1
        return self.seq


class FusedPeerExchange(PeerExchange):
    """PeerExchange whose two halves run inside the batch-norm kernels: the kernel that finishes a
    reduction publishes the sums, the kernel that consumes them waits for all ranks in its prologue.
    No launch of its own; ShardedBatchNormAct picks the *_publish / *_peer entry points when it sees it."""
    fused = True


class InLaunchExchange:
    """The exchange of the single-launch sharded entry points (nnf_bn_train_fwd_sharded / _bwd_sharded): every
    rank owns a mailbox in symmetric memory; the launch that computes a channel's statistics stores them into
    all mailboxes and the same launch's apply work waits for them per channel. Nothing to call between
    kernels: ShardedBatchNormAct hands the mailbox pointers to the entry points. `all_reduce` (NCCL) is kept
    for the shapes those entry points do not take."""
    in_launch = True

    def __init__(self, kernels, channels, device, group=None):
        import os
        # plain peer loads/stores only: no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.k = kernels
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.channels = channels
        self.buf = symm_mem.empty(kernels.bn_train_mailbox_bytes(channels) // 8, dtype=torch.int64, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.seq = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)  # every mailbox is zeroed before anyone stores into it

    def next_seq(self):
        self.seq += 1
        return self.seq

    def all_reduce(self, tensor):
        dist.all_reduce(tensor, group=self.group)


class ExchangeTimeout(RuntimeError):
    """A single-launch sharded step gave up waiting for another rank's statistics (or for this GPU's own items): the
    outputs of that step are not to be used. `reports` holds the launch reports that said so."""

    def __init__(self, reports):
        super().__init__("a batch-sharded batch-norm launch ran out of its bounded wait: %s" % (reports,))
        self.reports = reports


class ShardedBatchNormAct:
    # A backend with nnf_set_error_sink raises one word of pinned host memory when a bounded wait runs out; the layers of a
    # process share it, so the one that finds it raised counts a failure for all of them.
    _process_sink = None
    _process_failures = 0

    def __init__(self, kernels, channels, eps, acts, device, group=None, on_phase=None, exchange=None):
        self.k = kernels
        self._sink = None
        if hasattr(kernels, "set_error_sink") and torch.cuda.is_available():
            if ShardedBatchNormAct._process_sink is None:
                word = torch.zeros(1, dtype=torch.int32).pin_memory()
                kernels.set_error_sink(word)
                ShardedBatchNormAct._process_sink = word
            self._sink = ShardedBatchNormAct._process_sink
        self._seen_failures = ShardedBatchNormAct._process_failures
        self._launched = {}       # direction -> workspace of this layer's most recent single launch
        self._pending = []        # (event, pinned report words, what) of single-launch steps not yet looked at
        self._free_reports = []
        self.degraded = False     # after a timed-out step: the NCCL sequence until reset_exchange()
        self.exchange = exchange if exchange is not None else NcclExchange(group)
        self.on_phase = on_phase or (lambda name: None)  # called after each enqueue, e.g. to record CUDA events
        self.c = channels
        self.eps = eps
        self.acts = list(acts)
        self.group = group
        self.world = _world(group)
        f = dict(dtype=torch.float32, device=device)
        self.sums = torch.zeros(2 * channels, **f)     # forward message
        self.saved = torch.zeros(2 * channels, **f)    # {mean, invstd}: the reference's temporary_fixed_buffer
        self.bsums = torch.zeros(3 * channels, **f)    # local {sum du, sum du*xhat, sum dslope}
        self.gsums = torch.zeros(2 * channels, **f)    # backward message
        # one workspace per direction: a launch's report sits at the head of its workspace until the next launch in the same
        # direction clears it, a whole step later, so the copy of the report to the host can run beside the main stream
        self.workspaces = {}
        self._report_copied = {}   # direction -> event after which that direction's workspace may be cleared again
        self._side = None
        self._marks = {}
        self._shape_ok = {}

    def _ws(self, x, which="forward"):
        n, c = x.shape[0], x.shape[1]
        hw = x.numel() // max(n * c, 1)
        need = self.k.bn_train_workspace_bytes(n, c, hw)
        ws = self.workspaces.get(which)
        if ws is None or ws.numel() < need:
            ws = self.workspaces[which] = torch.empty(need, dtype=torch.uint8, device=x.device)
        copied = self._report_copied.pop(which, None)
        if copied is not None:
            torch.cuda.current_stream().wait_event(copied)   # long done by now: costs nothing on the device
        return ws

    def count_total(self, x, global_entries=None):
        n, c = x.shape[0], x.shape[1]
        hw = x.numel() // max(n * c, 1)
        entries = global_entries if global_entries is not None else n * self.world
        return float(entries * hw)

    # ---- what the single-launch steps report ------------------------------------------------------------------
    def _note_launch(self, what, workspace):
        """With a host-visible error word: nothing is added to the stream, the launch's workspace is remembered so that its report
        can be fetched if the word is ever raised. Otherwise enqueues the copy of the launch's report behind the launch; looked at
        by check()."""
        read = getattr(self.k, "read_report", None)
        if read is None:
            return
        if self._sink is not None:
            self._launched[what] = workspace
            return
        words = self._free_reports.pop() if self._free_reports else self._new_report()
        if hasattr(self.k, "make_event"):      # a backend without streams (the CPU tests)
            read(words, workspace)
            event = self.k.make_event()
            event.record()
        else:
            # beside the main stream: a 256-byte device-to-host copy between two launches of the main stream would hold the
            # second launch back by about ten microseconds (two GPUs: 295 us per step with it, 269 us without)
            if self._side is None:
                self._side = torch.cuda.Stream()
            marks = self._marks.get(what)
            if marks is None:   # two events per direction, recorded again at every launch
                marks = self._marks[what] = (torch.cuda.Event(), torch.cuda.Event())
            launched, event = marks
            launched.record()
            self._side.wait_event(launched)
            read(words, workspace, stream=self._side)
            event.record(self._side)
            self._report_copied[what] = event
        self._pending.append((event, words, what))

    def _new_report(self):
        words = torch.zeros(self.k.REPORT_WORDS, dtype=torch.int64)
        return words.pin_memory() if torch.cuda.is_available() else words

    def check(self, block=True):
        """Looks at the reports of the single-launch steps enqueued so far (all of them with block=True, else those the
        GPU has already finished). A step whose wait ran out raises ExchangeTimeout; from then on the layer runs the
        statistics kernel / NCCL all-reduce / apply kernel sequence, which cannot time out silently, until
        reset_exchange() is called. Call it at a step boundary, before the outputs of the step are trusted."""
        if self._sink is not None:
            if block:
                torch.cuda.current_stream().synchronize()
            if int(self._sink[0]) != 0:
                # some launch of this process gave up a wait: find out whether it was one of this layer's, tell every layer
                torch.cuda.synchronize()
                code = int(self._sink[0])
                self._sink[0] = 0
                ShardedBatchNormAct._process_failures += 1
                self._last_failure = [(what, r) for what, r in self._fetch_reports() if r["status"] != 0] or [("a launch of this process", {"status": code})]
            if self._seen_failures != ShardedBatchNormAct._process_failures:
                self._seen_failures = ShardedBatchNormAct._process_failures
                self.degraded = True
                raise ExchangeTimeout(getattr(self, "_last_failure", [("a launch of this process", {"status": -1})]))
            return
        bad, still = [], []
        for event, words, what in self._pending:
            if not block and not event.query():
                still.append((event, words, what))
                continue
            event.synchronize()
            report = self.k.parse_report(words)
            self._free_reports.append(words)
            if report["status"] != 0:
                bad.append((what, report))
        self._pending = still
        if bad:
            self.degraded = True
            raise ExchangeTimeout(bad)

    def reset_exchange(self):
        self.degraded = False

    def _fetch_reports(self):
        """The reports of this layer's most recent launch in each direction, read now (synchronises the device)."""
        out = []
        for what, workspace in self._launched.items():
            words = self._new_report()
            self.k.read_report(words, workspace)
            torch.cuda.synchronize()
            out.append((what, self.k.parse_report(words)))
        return out

    def last_wait_ns(self):
        """(sum, max) of the waits inside the most recent single-launch step whose report has arrived; (0, 0) if none."""
        total = longest = 0
        if self._sink is not None:
            for what, r in self._fetch_reports():
                total, longest = total + r["wait_ns_total"], max(longest, r["wait_ns_max"])
            return total, longest
        for event, words, what in self._pending:
            if event.query():
                r = self.k.parse_report(words)
                total, longest = total + r["wait_ns_total"], max(longest, r["wait_ns_max"])
        return total, longest

    def _in_launch_ok(self, x, hw):
        """Shapes the one-launch sharded entry points take (the library decides; planes of whole float4s always are)."""
        key = (x.shape[0], x.shape[1], hw)
        if key not in self._shape_ok:
            supported = getattr(self.k, "bn_train_sharded_supported", None)
            self._shape_ok[key] = bool(supported(*key)) if supported is not None else hw % 4 == 0
        return self._shape_ok[key]

    def forward(self, y, x, gamma, beta, global_entries=None):
        m = self.count_total(x, global_entries)
        self.on_phase("start")
        ex = self.exchange
        hw = x.numel() // max(x.shape[0] * x.shape[1], 1)
        if self._pending or self._sink is not None:
            self.check(block=False)
        if self.world > 1 and getattr(ex, "in_launch", False) and not self.degraded and self._in_launch_ok(x, hw) and x.shape[1] == ex.channels:
            ws = self._ws(x, "forward")
            self.k.bn_train_fwd_sharded(y, self.saved, self.sums, x, gamma, beta, self.eps, self.acts, m, ws, ex.ptrs, ex.rank, ex.world,
                                        ex.next_seq())
            self._note_launch("forward", ws)
            self.on_phase("stats")
            self.on_phase("allreduce_fwd")
            self.on_phase("apply")
            return y
        if self.world > 1 and getattr(ex, "fused", False) and not self.degraded and hw % 4 == 0:
            seq = ex.next_seq()
            self.k.bn_train_stats_publish(self.sums, x, self._ws(x), ex.ptrs, ex.rank, ex.world, ex.kmax, seq)
            self.on_phase("stats")
            self.on_phase("allreduce_fwd")
            self.k.bn_train_apply_act_peer(y, self.saved, x, gamma, beta, ex.buf, ex.world, ex.kmax, seq, m, self.eps, self.acts)
            self.on_phase("apply")
            return y
        self.k.bn_train_stats(self.sums, x, self._ws(x))
        self.on_phase("stats")
        if self.world > 1:
            ex.all_reduce(self.sums)
        self.on_phase("allreduce_fwd")
        self.k.bn_train_apply_act(y, self.saved, x, gamma, beta, self.sums, m, self.eps, self.acts)
        self.on_phase("apply")
        return y

    def backward(self, dx, dy, x, gamma, beta, grads=None, running=None, global_entries=None, add_to_destination=False):
        """grads: dict with optional 'gamma', 'beta', 'slope', 'mean', 'invsigma' accumulators;
        running: (mean, invsigma) when the running-statistics pseudo-gradients are wanted."""
        m = self.count_total(x, global_entries)
        grads = grads or {}
        sharded = self.world > 1
        mean, invsigma = running if running is not None else (None, None)
        ex = self.exchange
        hw = x.numel() // max(x.shape[0] * x.shape[1], 1)
        if sharded and getattr(ex, "in_launch", False) and not self.degraded and self._in_launch_ok(x, hw) and x.shape[1] == ex.channels and not add_to_destination:
            self.on_phase("bwd_stats")
            ws = self._ws(x, "backward")
            self.k.bn_train_bwd_sharded(dx, self.bsums, dy, x, gamma, beta, self.saved, self.acts, m, ws, ex.ptrs, ex.rank, ex.world,
                                        ex.next_seq(), grad_gamma=grads.get("gamma"), grad_beta=grads.get("beta"), grad_mean=grads.get("mean"),
                                        grad_invsigma=grads.get("invsigma"), grad_slope=grads.get("slope"), mean=mean, invsigma=invsigma,
                                        entry_count=float(x.shape[0]))
            self._note_launch("backward", ws)
            self.on_phase("allreduce_bwd")
            self.on_phase("bwd_apply")
            return dx
        if sharded and getattr(ex, "fused", False) and not self.degraded:
            seq = ex.next_seq()
            self.k.bn_train_bwd_stats_publish(self.bsums, dy, x, gamma, beta, self.saved, self.acts, self._ws(x), ex.ptrs, ex.rank, ex.world, ex.kmax, seq)
            self.on_phase("bwd_stats")
            self.on_phase("allreduce_bwd")
            self.k.bn_train_bwd_apply_peer(dx, dy, x, gamma, beta, self.saved, ex.buf, ex.world, ex.kmax, seq, self.bsums, m, self.acts,
                                           grad_gamma=grads.get("gamma"), grad_beta=grads.get("beta"), grad_mean=grads.get("mean"),
                                           grad_invsigma=grads.get("invsigma"), grad_slope=grads.get("slope"), mean=mean, invsigma=invsigma,
                                           entry_count=float(x.shape[0]), add_to_destination=add_to_destination)
            self.on_phase("bwd_apply")
            return dx
        self.k.bn_train_bwd_stats(self.bsums, dy, x, gamma, beta, self.saved, self.acts, self._ws(x), gsums=self.gsums if sharded else None)
        self.on_phase("bwd_stats")
        if sharded:
            self.exchange.all_reduce(self.gsums)
        self.on_phase("allreduce_bwd")
        mean, invsigma = running if running is not None else (None, None)
        self.k.bn_train_bwd_apply(dx, dy, x, gamma, beta, self.saved, self.gsums if sharded else self.bsums, self.bsums, m, self.acts,
                                  grad_gamma=grads.get("gamma"), grad_beta=grads.get("beta"), grad_mean=grads.get("mean"),
                                  grad_invsigma=grads.get("invsigma"), grad_slope=grads.get("slope"), mean=mean, invsigma=invsigma,
                                  entry_count=float(x.shape[0]), add_to_destination=add_to_destination)
        self.on_phase("bwd_apply")
        return dx
