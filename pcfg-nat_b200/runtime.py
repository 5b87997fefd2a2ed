"""Fixed-shape steps of the structured-loss / decoding path, replayable as CUDA graphs.

Each step is what the reference's Python does around the custom operators for one batch:

* ``LossStep``   — training (fs_plugins/criterions/nat_pcfg_loss.py:98-135): emissions of the targets from
  the decoder states (fused projection, EOS masking included), PCFG loss with both gradients, and the
  three statistics the scalar loss is formed from;
* ``GlanceStep`` — glancing pass (nat_pcfg_loss.py:193-227): emissions + arg-max tokens, inside table,
  best-tree alignment;
* ``DecodeStep`` — Viterbi inference (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:483-502):
  max log-prob / arg-max token per node, Viterbi tables, length-penalised choice of the output length,
  back-trace on the device.

A step launches a handful of small-to-medium kernels whose device time (~1 ms at training-batch size) is
of the order of the host cost of enqueueing them through Python, so it is captured once into CUDA graphs
and replayed.  Inputs live in static device buffers; ``load`` copies a new batch into them (from pinned
host memory or from device tensors).

A step has two stages, each its own graph: the projection, which reads the decoder states, and the
dynamic program, which reads the transition matrix (the larger input).  ``load(..., overlap=True)`` sends
the inputs over a copy stream in that order and ``run`` lets each stage wait only for its own inputs, so
that the transitions are still in flight from the host while the projection runs.  The decoder states
themselves are sent in ``copy_chunks`` groups of sentences, each projected (by a graph of its own) as soon
as it has landed, so that only the first group's copy is not hidden behind the tensor cores.
"""
import torch

from . import sharding
from .custom_ops import pcfg_loss as ops


class _GraphedStep:
    def __init__(self, weight, B, L, device, use_graph=True, copy_chunks=2):
        if weight.dtype != torch.float16 or not weight.is_cuda:
            raise RuntimeError("weight must be a float16 CUDA tensor [V, H]")
        self.device = torch.device(device)
        self.weight = weight.contiguous()
        self.V, self.H = weight.shape
        self.B, self.L = B, L
        dev = self.device
        self.hidden = torch.zeros((B, L, self.H), dtype=torch.float16, device=dev)
        self.links = torch.full((B, L, 2, L), float("-inf"), dtype=torch.float32, device=dev)
        self.output_length = torch.full((B,), 2, dtype=torch.int64, device=dev)
        self.use_graph = use_graph
        self.graphs = None
        self.mid = None
        self.out = None
        self.kernel = ops.get_pcfg_kernel()
        self.copy_stream = None
        self._ev_stage1 = self._ev_stage2 = self._ev_done = None
        self._ev_ran = None  # end of this object's last run(): the point after which its input buffers are free
        self._pending = False
        self._pending_chunked = False
        self.last_load_bytes = None
        # How an overlapped load takes the large inputs from pinned host memory.  None: copy engines only (the padded
        # states and the main-chain rows of the transitions; copies overlap the kernels of the previous batch
        # completely).  "links": the transitions by a kernel that reads the host buffer itself and fetches only the
        # entries the tree masks leave finite (a quarter of the bytes of the main-chain rows); "all": the states of
        # the real graph nodes that way too.  A fetching kernel needs SMs, which the persistent compute kernels do not
        # share, so it pays where the bus is the bottleneck (several GPUs pulling from one host), not on one GPU.
        self.fetch_from_host = None
        # an overlapped load from pinned host memory, with the lengths in host memory too, sends the decoder states of
        # the real graph nodes and skips most padding rows (which are never read): at most this many copy-engine
        # copies per sentence group, joined across the smallest gaps; 0 = the whole padded tensor in one copy per
        # group.  A copy costs the host 5 to 7 us and the copy engine its set-up: on a training batch 8 per group
        # measured best (0.512 ms per step against 0.519 with 0, 0.550 with 16, 0.658 with 32)
        self.copy_real_rows = 8
        # sentence groups [b0, b1) of an overlapped load; chunking needs the graphs (it is a replay trick)
        n = max(1, min(int(copy_chunks), B)) if use_graph else 1
        self.chunks = [(B * i // n, B * (i + 1) // n) for i in range(n)]
        self.chunk_graphs = None
        self._ev_chunk = None
        # after an overlapped load: project sentence group by sentence group as the groups arrive (pays when the step
        # waits for its own copies), or the whole batch at once when the copies are long done (a pipeline of steps)
        self.project_by_group = True

    def _inputs(self):
        return [self.hidden, self.links, self.output_length]

    def _stage2_inputs(self):
        """The inputs only the second stage reads (sent last by an overlapped load)."""
        return [self.links]

    def input_bytes(self):
        """Bytes one ``load`` moves.  After an overlapped load from pinned host memory: what that load fetched (the
        decoder states of the real nodes and the transitions the kernels read, see ``load``).  Otherwise every input
        whole, except the transitions, of which only the rows of main-chain nodes (every other row) are copied."""
        if self.last_load_bytes is not None:
            return self.last_load_bytes
        return sum(t.numel() * t.element_size() // (2 if t is self.links else 1) for t in self._inputs())

    def _fetched_bytes(self, tensors, lengths, fetch_hidden, fetch_links, hidden_rows_copied=None):
        """Bytes an overlapped load moves for sentences of ``lengths`` graph nodes when a kernel fetches the states
        and / or the transitions from the host buffers, or when ``hidden_rows_copied`` rows of the states went by
        copy engine."""
        bufs = self._inputs()
        m = lengths.clamp(max=self.L).double()
        total = 0.0
        for dst, src in zip(bufs, tensors):
            if dst is self.hidden and hidden_rows_copied is not None:
                total += float(hidden_rows_copied) * self.H * 2
            elif dst is self.hidden and fetch_hidden:
                total += float(m.sum()) * self.H * 2
            elif dst is self.links and fetch_links:
                # main-chain nodes a = 1, 3, .. < m, both left options, columns a + 1 .. m - 1
                k = torch.floor(m / 2)  # their number; sum over them of (m - 1 - a) = k (m - 1) - k^2
                total += float((2 * 4 * (k * (m - 1) - k * k)).clamp(min=0).sum())
            elif dst is self.links:
                total += src.numel() * src.element_size() // 2  # the strided copy of the main-chain rows
            else:
                total += src.numel() * src.element_size()
        return int(total)

    def _copy_in(self, dst, src):
        if dst is self.links and src.dtype == torch.float32 and src.is_contiguous() and dst.shape[1] % 2 == 0 \
                and tuple(src.shape) == tuple(dst.shape):
            self.kernel.copy_links_main_rows(dst, src)  # the other rows stay -inf, as the constructor left them
        else:
            dst.copy_(src, non_blocking=True)

    def load(self, *tensors, overlap=False):
        """Copies one batch into the static buffers; same order as ``_inputs``.

        overlap=False: asynchronous copies on the current stream.  overlap=True: on the step's copy stream,
        first-stage inputs first; the next ``run`` orders each stage after the arrival of its own inputs and
        the copies after this object's previous ``run`` (which still reads the buffers).  From pinned host tensors
        an overlapped load sends the decoder states of the real graph nodes and skips most of the padding rows
        (``copy_real_rows`` copies per sentence group) and the main-chain rows of the transitions; with ``fetch_from_host`` a kernel reads the host
        buffers instead and moves only what the kernels read: the states of the real nodes ("all"), and of the
        transitions the entries links[a][k][c] with a on the main chain and a < c < m_b ("links", "all") — everything
        the model's tree masks leave finite; the rest of those rows is -inf in the step's buffer."""
        bufs = self._inputs()
        if len(tensors) != len(bufs):
            raise RuntimeError(f"expected {len(bufs)} tensors")
        if not overlap:
            for dst, src in zip(bufs, tensors):
                self._copy_in(dst, src)
            return
        if self.copy_stream is None:
            self.copy_stream = torch.cuda.Stream(self.device)
            self._ev_stage1, self._ev_stage2, self._ev_done = (torch.cuda.Event() for _ in range(3))
            self._ev_chunk = [torch.cuda.Event() for _ in self.chunks]
        late = {id(t) for t in self._stage2_inputs()}
        with torch.cuda.stream(self.copy_stream):
            # the buffers are free once this object's own last run has read them; work queued since then on the
            # current stream (another step object's run, say) does not hold the copies back
            if self._ev_ran is not None:
                self.copy_stream.wait_event(self._ev_ran)
            else:  # never run yet: after whatever initialised the buffers on the current stream
                self._ev_done.record(torch.cuda.current_stream(self.device))
                self.copy_stream.wait_event(self._ev_done)
            for dst, src in zip(bufs, tensors):  # the small inputs first, then the states group by group
                if id(dst) not in late and dst is not self.hidden:
                    self._copy_in(dst, src)
            src_of = {id(dst): src for dst, src in zip(bufs, tensors)}
            src_hidden = src_of[id(self.hidden)]
            src_links = src_of.get(id(self.links))
            pinned = lambda t, buf: t is not None and not t.is_cuda and t.is_pinned() and t.dtype == buf.dtype and \
                tuple(t.shape) == tuple(buf.shape)
            fetch = self.fetch_from_host == "all" and pinned(src_hidden, self.hidden)
            src_len = src_of[id(self.output_length)]
            rows_only = (not fetch and self.copy_real_rows and pinned(src_hidden, self.hidden) and not src_len.is_cuda
                         and src_len.dtype == torch.int64 and src_len.is_contiguous())
            if fetch:  # one kernel reads the real nodes' states from the host buffer
                self.kernel.stage_inputs(self.output_length, hidden_dst=self.hidden, hidden_src=src_hidden)
                for ev in self._ev_chunk:
                    ev.record(self.copy_stream)
            else:
                rows_sent = 0
                for (b0, b1), ev in zip(self.chunks, self._ev_chunk):
                    if rows_only:  # the states of the real nodes and the padding rows of the narrowest gaps
                        rows_sent += self.kernel.copy_real_rows(self.hidden, src_hidden, src_len, b0, b1,
                                                                max_copies=int(self.copy_real_rows))
                    else:
                        self.hidden[b0:b1].copy_(src_hidden[b0:b1], non_blocking=True)
                    ev.record(self.copy_stream)
            self._ev_stage1.record(self.copy_stream)
            fetch_links = self.fetch_from_host in ("links", "all") and id(self.links) in late and pinned(src_links, self.links)
            for dst, src in zip(bufs, tensors):
                if id(dst) in late:
                    if dst is self.links and fetch_links:  # the transitions the tree masks leave finite, nothing else
                        self.kernel.stage_inputs(self.output_length, links_dst=self.links, links_src=src)
                    else:
                        self._copy_in(dst, src)
            self._ev_stage2.record(self.copy_stream)
            self.last_load_bytes = None
            if fetch or fetch_links or rows_only:
                lengths = src_of[id(self.output_length)].cpu()
                self.last_load_bytes = self._fetched_bytes(tensors, lengths, fetch, fetch_links,
                                                           rows_sent if rows_only else None)
        self._pending = True
        self._pending_chunked = not fetch

    def _stage1(self, b0=0, b1=None):
        """The projection of sentences [b0, b1) (all of them by default): a dict of [b1 - b0, ...] tensors."""
        raise NotImplementedError

    def _stage2(self, mid):
        raise NotImplementedError

    def _capture(self):
        # warm up on a side stream (lazy module loading, allocator), then capture one graph per stage
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._stage2(self._stage1())
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g1):
            self.mid = self._stage1()
        with torch.cuda.graph(g2, pool=g1.pool()):
            self.out = self._stage2(self.mid)
        self.graphs = (g1, g2)
        self.chunk_graphs = []
        if len(self.chunks) > 1:  # the first stage once more, group by group, writing into the same tensors
            for b0, b1 in self.chunks:
                with torch.cuda.stream(s):
                    self._stage1(b0, b1)
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=g1.pool()):
                    part = self._stage1(b0, b1)
                    for key, val in part.items():
                        self.mid[key][b0:b1].copy_(val)
                self.chunk_graphs.append(g)

    def run(self):
        cur = torch.cuda.current_stream(self.device)
        pending, self._pending = self._pending, False
        if self.use_graph and self.graphs is None:
            if pending:  # capture must not race the copies
                cur.wait_event(self._ev_stage2)
                pending = False
            self._capture()
        if pending and self.chunk_graphs and self._pending_chunked and self.project_by_group:
            for ev, g in zip(self._ev_chunk, self.chunk_graphs):
                cur.wait_event(ev)
                g.replay()
        else:
            if pending:
                cur.wait_event(self._ev_stage1)
            if self.use_graph:
                self.graphs[0].replay()
            else:
                self.mid = self._stage1()
        if pending:
            cur.wait_event(self._ev_stage2)
        if self.use_graph:
            self.graphs[1].replay()
        else:
            self.out = self._stage2(self.mid)
        if self._ev_ran is None:
            self._ev_ran = torch.cuda.Event()
        self._ev_ran.record(cur)
        return self.out


class PipelinedStep:
    """Several step objects of the same shape (two by default) used in turn, so that the host-to-device copies of the
    next batches run while batch i is computed (each object has its own static buffers and graphs): ``load`` always
    goes over the copy stream of the object whose turn it is and waits only for that object's previous run, ``depth``
    batches back.  ``run`` returns that object's static outputs, which stay valid until ``depth`` - 1 more runs."""

    def __init__(self, make_step, fetch_from_host=None, depth=2):
        if depth < 2:
            raise ValueError("a pipeline needs at least two step objects")
        self.steps = [make_step() for _ in range(depth)]
        for st in self.steps:
            st.fetch_from_host = fetch_from_host
            st.project_by_group = False  # a batch's copies ran under the previous batch's kernels: nothing to wait for
        self.turn = 0

    def load(self, *tensors):
        self.steps[self.turn].load(*tensors, overlap=True)

    def run(self):
        out = self.steps[self.turn].run()
        self.turn = (self.turn + 1) % len(self.steps)
        return out

    def input_bytes(self):
        return self.steps[self.turn - 1].input_bytes()  # of the batch loaded last

    @property
    def kernels_per_step(self):
        return self.steps[0].kernels_per_step


class LossStep(_GraphedStep):
    """projection -> loss forward+backward -> loss statistics for fixed (B, L, T, H, V).

    Inputs (``load`` order): hidden [B,L,H] f16, links [B,L,2,L] f32, output_length [B], targets [B,T],
    target_length [B].  ``run()`` returns (stats[3] f32 = [sum_b S_b/n_b, sentences, invalid],
    match_all_grad, links_grad, sentence_loss); static outputs, overwritten by the next ``run()``.
    With ``link_features`` the transitions are formed from the projected link features inside the step and the
    third output is the tuple of their gradients (see the constructor).
    """
    kernels_per_step = 7  # proj_prepare, proj, proj_merge, loss_fwd, outside, grad, loss_stats (set per shape below)

    def __init__(self, weight, B, L, T, device, use_graph=True, copy_chunks=2, proj_backward=False, exchange=None,
                 force_emit=False, link_features=None, left_tree_mask=None, right_tree_mask=None, main_chain=None,
                 pad_index=1):
        super().__init__(weight, B, L, device, use_graph, copy_chunks)
        self.T = T
        # link_features=(heads, head_dim): the step takes the projected link features instead of the transition
        # matrix (inputs query, key_left, key_right [B,L,heads,head_dim] f16, gate_logits [B,L,heads] f32,
        # prev_output_tokens [B,L] in place of links), forms the transitions itself (the model's extract_links,
        # models/...pcfg.py:140-201) and carries the loss gradient back to the features: run() then returns d query,
        # d key_left, d key_right, d gate_logits in place of links_grad.  The three tree masks are needed.
        self.link_features = link_features
        if link_features is not None:
            heads, dim = link_features
            dev = self.device
            self.pad_index = int(pad_index)
            self.query, self.key_left, self.key_right = (torch.zeros((B, L, heads, dim), dtype=torch.float16, device=dev)
                                                         for _ in range(3))
            self.gate_logits = torch.zeros((B, L, heads), dtype=torch.float32, device=dev)
            self.prev_output_tokens = torch.full((B, L), self.pad_index, dtype=torch.int64, device=dev)
            u8 = lambda t: t.to(dev).ne(0).to(torch.uint8).contiguous()
            self.left_u8, self.right_u8 = u8(left_tree_mask[:L, :L]), u8(right_tree_mask[:L, :L])
            self.main_u8 = u8(main_chain[:L])
        # force_emit: the training pass after a glancing pass (criterions/nat_pcfg_loss.py:116-121): two more
        # inputs, matchmask [B,T,L] and keep_word_mask [B,L] (bool, as GlanceStep returns them); a revealed node
        # may only emit its aligned target position and gets no gradient
        self.force_emit = bool(force_emit)
        if self.force_emit:
            self.matchmask = torch.zeros((B, T, L), dtype=torch.bool, device=self.device)
            self.keep_word_mask = torch.zeros((B, L), dtype=torch.bool, device=self.device)
        # a sharding.LossExchange: the statistics come back summed over the ranks of the job (same launch)
        self.exchange = exchange
        self.targets = torch.zeros((B, T), dtype=torch.int64, device=self.device)
        self.target_length = torch.ones((B,), dtype=torch.int64, device=self.device)
        # with proj_backward the step also carries the emission gradients back through the projection:
        # run() then returns d hidden [B,L,H] f16 and d weight [V,H] f16 as two more outputs
        self.proj_backward = bool(proj_backward)
        if type(self) is LossStep:
            # the library says whether the outside pass of this shape also sums up the gradients (2 DP kernels) or
            # a gradient kernel follows it (3); around them: proj_prepare, proj, proj_merge and loss_stats
            from . import _cabi
            with torch.cuda.device(self.device):
                dp = _cabi.lib().pcfgnat_loss_fwd_bwd_kernels(B, L, T, 1)
            # with link features: feature gather, score products, links, and the two backward kernels
            self.kernels_per_step = 4 + (dp if dp > 0 else 3) + (2 if self.force_emit else 0) + (5 if link_features else 0)
        self.proj_backward_note = None
        if self.proj_backward:
            self.kernels_per_step += 5  # proj_prepare, row index, proj (grad mode), the two products of the backward
            self.weight_bf16 = self.weight.to(torch.bfloat16)
            V = int(self.weight.shape[0])
            # d-logits of the real graph nodes only, compact; the two GEMMs run after the graph, over as many rows
            # as the batch has real nodes (a number the host knows from the lengths it loaded)
            self.dlogits = torch.empty((B * L, V), dtype=torch.bfloat16, device=self.device)
            self.row_index = torch.zeros((B * L,), dtype=torch.int64, device=self.device)
            self.d_hidden = torch.zeros((B * L, self.H), dtype=torch.float16, device=self.device)
            self.n_rows = None
            self.proj_backward_note = ("the step plus d hidden and d weight of the projection: logits recomputed into "
                                       "bf16 d-logits of the real graph nodes by proj_kernel's gradient mode (in the "
                                       "graph), then this library's two tcgen05 products over those rows (launched "
                                       "after the graph: their row count changes from batch to batch)")

    def _inputs(self):
        if self.link_features is not None:
            base = [self.hidden, self.query, self.key_left, self.key_right, self.gate_logits, self.prev_output_tokens,
                    self.output_length, self.targets, self.target_length]
        else:
            base = [self.hidden, self.links, self.output_length, self.targets, self.target_length]
        return base + ([self.matchmask, self.keep_word_mask] if self.force_emit else [])

    def _stage2_inputs(self):
        if self.link_features is None:
            return super()._stage2_inputs()
        return [self.query, self.key_left, self.key_right, self.gate_logits, self.prev_output_tokens]

    def _stage1(self, b0=0, b1=None):
        return self.kernel.proj_logsoftmax_gather(self.hidden[b0:b1], self.weight, self.targets[b0:b1],
                                                  self.output_length[b0:b1], self.target_length[b0:b1],
                                                  want_lse=self.proj_backward)

    def _stage2(self, em):
        if self.force_emit:
            self.kernel.force_emit(em["match"], self.matchmask, self.keep_word_mask, out=em["match"])
        links, saved = self.links, None
        if self.link_features is not None:
            links, saved = self.kernel._links_forward(self.query, self.key_left, self.key_right, self.gate_logits,
                                                      self.prev_output_tokens, self.pad_index, self.left_u8, self.right_u8,
                                                      self.main_u8)
        loss, mg, lg = self.kernel.pcfg_loss_fwd_bwd(em["match"], links, self.output_length, self.target_length)
        if self.force_emit:
            self.kernel.force_emit_grad(mg, self.keep_word_mask, out=mg)
        if saved is not None:
            lg = self.kernel._links_backward(lg, saved)  # (d query, d key_left, d key_right, d gate_logits), float32
        stats = (self.exchange.stats(loss, self.target_length) if self.exchange is not None
                 else sharding.local_loss_stats(loss, self.target_length))
        if not self.proj_backward:
            return stats, mg, lg, loss
        self.kernel.proj_dlogits(self.hidden, self.weight, self.targets, self.output_length, self.target_length,
                                 em["lse"], mg, n_rows=self.B * self.L, out=self.dlogits, row_index_out=self.row_index)
        return stats, mg, lg, loss

    def load(self, *tensors, overlap=False):
        super().load(*tensors, overlap=overlap)
        if self.proj_backward:
            lengths = next(t for buf, t in zip(self._inputs(), tensors) if buf is self.output_length)
            # lengths in host memory: the row count of the backward GEMMs without a device read
            self.n_rows = None if lengths.is_cuda else int(lengths.clamp(min=0, max=self.L).sum())

    def run(self):
        out = super().run()
        if not self.proj_backward:
            return out
        n = self.n_rows if self.n_rows is not None else int(self.output_length.clamp(min=0, max=self.L).sum())
        dl, idx = self.dlogits[:n], self.row_index[:n]
        rows = self.hidden.view(self.B * self.L, self.H).index_select(0, idx)
        d_rows, d_weight = ops.proj_backward_products(dl, self.weight_bf16, rows)
        self.d_hidden.zero_()
        self.d_hidden.index_copy_(0, idx, d_rows.to(torch.float16))
        d_weight = d_weight.to(torch.float16)
        self._ev_ran.record(torch.cuda.current_stream(self.device))  # the GEMMs still read the step's buffers
        return (*out, self.d_hidden.view(self.B, self.L, self.H), d_weight)


class GlanceStep(LossStep):
    """projection (emissions + arg-max tokens) -> inside table -> best tree -> glancing sampler.

    Inputs (``load`` order): those of ``LossStep`` and prev_output_tokens [B,L] int64.  ``run()`` returns
    (tree [B,L] i64, sentence log-likelihood [B], arg-max tokens [B,L] i64, sampler outputs: the dict of
    ``glance_select`` — match mask, oracle tokens, kept positions, decoder input of the second pass).  The
    sampler's normal draws are made inside the step into ``self.noise``."""
    kernels_per_step = 6  # proj_prepare, proj, proj_merge, loss_fwd, best_tree, glance_select

    def __init__(self, weight, B, L, T, device, use_graph=True, context_p=0.5, copy_chunks=2,
                 strategy="number-random"):
        super().__init__(weight, B, L, T, device, use_graph, copy_chunks)
        self.context_p = float(context_p)
        self.strategy = strategy  # the criterion's --glance-strategy: "number-random", "cmlm" or None
        self.prev_output_tokens = torch.ones((B, L), dtype=torch.int64, device=self.device)
        self.noise = torch.zeros((B, L), dtype=torch.float32, device=self.device)
        self.uniform = None
        if strategy == "cmlm":
            self.uniform = torch.zeros((B,), dtype=torch.float32, device=self.device)
        elif strategy is None:
            self.uniform = torch.zeros((B, L), dtype=torch.float32, device=self.device)

    def _inputs(self):
        return super()._inputs() + [self.prev_output_tokens]

    def _stage1(self, b0=0, b1=None):
        return self.kernel.proj_logsoftmax_gather(self.hidden[b0:b1], self.weight, self.targets[b0:b1],
                                                  self.output_length[b0:b1], self.target_length[b0:b1], want_max=True)

    def _stage2(self, em):
        k = self.kernel
        S, _ = k.pcfg_loss(em["match"], self.links, self.output_length, self.target_length, 1, want_c=False)
        tree = k.pcfg_best_tree(S, None, em["match"], self.links, self.output_length, self.target_length, 1)
        if self.strategy is not None:
            self.noise.normal_()
        if self.uniform is not None:
            self.uniform.uniform_()
        glance = k.glance_select(tree, em["argmax"], self.targets, self.prev_output_tokens, self.target_length,
                                 self.noise, self.context_p, self.strategy, self.uniform)
        return tree, S[:, 0, 0], em["argmax"], glance


class DecodeStep(_GraphedStep):
    """projection (max log-prob + arg-max token per node) -> Viterbi tables -> output length -> back-trace.

    Inputs (``load`` order): hidden, links, output_length.  ``run()`` returns (tokens [B,L] i64 padded with
    ``pad_index``, count [B] i64, predicted length [B] i64)."""
    kernels_per_step = 5  # proj_prepare, proj, proj_merge, viterbi, backtrace

    def __init__(self, weight, B, L, left_tree_mask, device, beta=1.0, pad_index=1, use_graph=True, copy_chunks=2,
                 link_features=None, right_tree_mask=None, main_chain=None, strategy="viterbi", decode_beta=1.0):
        """link_features=(heads, head_dim): the step takes the projected link features instead of the transition
        matrix and forms the latter itself (the model's extract_links, models/...pcfg.py:140-201).  Inputs
        (``load`` order) are then hidden, query, key_left, key_right [B,L,heads,head_dim] f16, gate_logits
        [B,L,heads] f32, prev_output_tokens [B,L] i64 and output_length; right_tree_mask and main_chain are needed."""
        super().__init__(weight, B, L, device, use_graph, copy_chunks)
        if strategy not in ("viterbi", "lookahead", "greedy"):
            raise RuntimeError(f"unknown decode strategy {strategy!r}")
        # the model's decode_strategy (models/...pcfg.py:419-502); "lookahead" weighs the children's best token
        # log-probabilities with decode_beta, "greedy" follows the transitions alone.  With these two ``run()``
        # returns (tokens, count) and no predicted length.
        self.strategy, self.decode_beta = strategy, float(decode_beta)
        if strategy != "viterbi":
            self.kernels_per_step = 4  # proj_prepare, proj, proj_merge, lookahead_decode
        self.mask = left_tree_mask.to(device=self.device, dtype=torch.int64).contiguous()
        self.pad_index = int(pad_index)
        # length penalty of the model: scores / arange(L // 4) ** beta (models/...pcfg.py:488-492)
        self.penalty = (torch.arange(L // 4, device=self.device) ** beta).to(torch.float32).unsqueeze(0)
        self.link_features = link_features
        if link_features is not None:
            heads, dim = link_features
            dev = self.device
            self.query, self.key_left, self.key_right = (torch.zeros((B, L, heads, dim), dtype=torch.float16, device=dev)
                                                         for _ in range(3))
            self.gate_logits = torch.zeros((B, L, heads), dtype=torch.float32, device=dev)
            self.prev_output_tokens = torch.full((B, L), self.pad_index, dtype=torch.int64, device=dev)
            u8 = lambda t: t.to(dev).ne(0).to(torch.uint8).contiguous()
            self.left_u8, self.right_u8 = u8(left_tree_mask[:L, :L]), u8(right_tree_mask[:L, :L])
            self.main_u8 = u8(main_chain[:L])

    def _inputs(self):
        if self.link_features is None:
            return super()._inputs()
        return [self.hidden, self.query, self.key_left, self.key_right, self.gate_logits, self.prev_output_tokens,
                self.output_length]

    def _stage2_inputs(self):
        if self.link_features is None:
            return super()._stage2_inputs()
        return [self.query, self.key_left, self.key_right, self.gate_logits, self.prev_output_tokens]

    def _stage1(self, b0=0, b1=None):
        return self.kernel.proj_logsoftmax_gather(self.hidden[b0:b1], self.weight, None, self.output_length[b0:b1], None,
                                                  want_max=True)

    def _stage2(self, em):
        k = self.kernel
        links = self.links
        if self.link_features is not None:
            links = k.extract_links(self.query, self.key_left, self.key_right, self.gate_logits, self.prev_output_tokens,
                                    self.pad_index, self.left_u8, self.right_u8, self.main_u8)
        if self.strategy != "viterbi":
            return k.lookahead_decode_device(links, em["max_lprob"], em["argmax"], self.output_length, self.mask,
                                             self.pad_index, self.decode_beta, self.strategy)
        S, R, Lt, Mt = k.pcfg_viterbi(em["max_lprob"], links, self.output_length, 1)
        tokens, count, pred = k.viterbi_decode_device(S, self.penalty, self.output_length, Lt, R, Mt, em["argmax"],
                                                      self.mask, self.pad_index)
        return tokens, count, pred
