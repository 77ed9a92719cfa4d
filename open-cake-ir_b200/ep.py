"""Expert-parallel FP8 MoE layer: tokens sharded T/R per rank, experts sharded E/R per rank
(rank r owns experts [r*E/R, (r+1)*E/R), the reference's ``local_expert_offset`` view,
src/open_cake_ir/tasks/solx_fib/moe.py:139-146), joined by an all-to-all dispatch and an
all-to-all combine over ``torch.distributed`` (NCCL over NVLink between GPUs; gloo in the CPU
tests of the exchange logic).

Per layer and rank:
  1. route the rank's own tokens (native routing kernel);
  2. for every destination rank that owns at least one of a token's experts, send the token ONCE:
     its e4m3 row, its K-block scales, its expert ids and route weights, packed into one byte row;
     one small all-to-all carries the per-rank row counts, one all-to-all the rows;
  3. run the rank-local layer on the received rows with routing given from outside -- pairs whose
     expert the rank does not own contribute nothing (moe.py:145-146) -- which yields, per received
     row, the bf16 sum of its local experts' weighted contributions;
  4. return those partial rows by the reverse all-to-all; the owner adds the at most R partial rows
     of a token in rank order in fp32 and rounds once to bf16.

The exchange plan is plain index arithmetic on the rank's device; ``route`` and ``local_layer`` are
injected so that the same class runs the native kernels on a GPU and the CPU oracle under gloo.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def exchange_plan(expert_ids: torch.Tensor, world: int, experts: int):
    """expert_ids int [T, K] -> (send_tokens [n] ordered by destination rank then token,
    send_counts [world], slot_of [T, world] = position of token t in the send list for rank r or -1)."""
    per_rank = experts // world
    dest = torch.div(expert_ids.long(), per_rank, rounding_mode="floor")
    ranks = torch.arange(world, device=expert_ids.device)
    needs = (dest[:, :, None] == ranks[None, None, :]).any(dim=1)          # [T, world]
    order = torch.nonzero(needs.t())                                      # rows (rank, token), rank-major
    send_tokens = order[:, 1]
    send_counts = needs.sum(dim=0)
    slot_of = torch.full(needs.shape, -1, dtype=torch.long, device=expert_ids.device)
    slot_of[order[:, 1], order[:, 0]] = torch.arange(order.shape[0], device=expert_ids.device)
    return send_tokens, send_counts, slot_of


def pack_rows(hidden_u8, hidden_scale, expert_ids, route_weights, tokens):
    """One byte row per sent token: H e4m3 bytes | H/128 fp32 scales | K int32 ids | K fp32 weights."""
    rows = hidden_u8[tokens]
    scales = hidden_scale.t()[tokens].contiguous().view(torch.uint8)
    ids = expert_ids[tokens].contiguous().view(torch.uint8)
    weights = route_weights[tokens].contiguous().view(torch.uint8)
    return torch.cat([rows, scales, ids, weights], dim=1).contiguous()


def row_bytes(hidden: int, top_k: int) -> int:
    return hidden + 4 * (hidden // 128) + 8 * top_k


class ExpertParallelMoe:
    """``forward()`` runs one layer over this rank's tokens.

    ``route(logits, bias, factor) -> (ids int32 [T,K], weights fp32 [T,K])`` and
    ``local_layer(hidden e4m3 [cap,H], scale fp32 [H/128,cap], ids int32 [cap,K], weights fp32 [cap,K])
    -> bf16 [cap,H]`` are the rank's routing and rank-local expert layer; ``capacity`` is the largest
    number of rows a rank can receive (the global token count)."""

    def __init__(self, *, experts: int, top_k: int, hidden: int, capacity: int, route, local_layer, group=None,
                 device="cuda"):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.experts, self.top_k, self.hidden, self.capacity = experts, top_k, hidden, capacity
        self.route, self.local_layer = route, local_layer
        self.device = torch.device(device)
        kb = hidden // 128
        self.recv_hidden = torch.zeros((capacity, hidden), dtype=torch.uint8, device=self.device)
        self.recv_scale = torch.zeros((kb, capacity), dtype=torch.float32, device=self.device)
        self.recv_ids = torch.full((capacity, top_k), -1, dtype=torch.int32, device=self.device)
        self.recv_weights = torch.zeros((capacity, top_k), dtype=torch.float32, device=self.device)
        self.last_counts = None

    def _all_to_all(self, out, inp, out_split, in_split):
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, out_split, in_split, group=self.group)

    def forward(self, routing_logits, routing_bias, routed_scaling_factor, hidden_states, hidden_states_scale):
        tokens = hidden_states.shape[0]
        kb = self.hidden // 128
        ids, weights = self.route(routing_logits, routing_bias, routed_scaling_factor)
        send_tokens, send_counts, slot_of = exchange_plan(ids, self.world, self.experts)
        recv_counts = torch.empty_like(send_counts)
        self._all_to_all(recv_counts, send_counts, None, None)
        counts = torch.stack([send_counts, recv_counts]).cpu()             # the one host sync of the layer
        send_split, recv_split = counts[0].tolist(), counts[1].tolist()
        n_send, n_recv = sum(send_split), sum(recv_split)
        if n_recv > self.capacity:
            raise RuntimeError("received more rows than the layer was sized for")
        self.last_counts = (send_split, recv_split)
        packed = pack_rows(hidden_states.view(torch.uint8), hidden_states_scale, ids, weights, send_tokens)
        width = row_bytes(self.hidden, self.top_k)
        received = torch.empty((n_recv, width), dtype=torch.uint8, device=self.device)
        self._all_to_all(received, packed, recv_split, send_split)
        # unpack into the rank-local layer's fixed-capacity inputs; unused rows keep expert id -1
        self.recv_ids.fill_(-1)
        self.recv_hidden[:n_recv] = received[:, :self.hidden]
        o = self.hidden
        self.recv_scale[:, :n_recv] = received[:, o:o + 4 * kb].contiguous().view(torch.float32).t()
        o += 4 * kb
        self.recv_ids[:n_recv] = received[:, o:o + 4 * self.top_k].contiguous().view(torch.int32)
        o += 4 * self.top_k
        self.recv_weights[:n_recv] = received[:, o:o + 4 * self.top_k].contiguous().view(torch.float32)
        partial = self.local_layer(self.recv_hidden.view(torch.float8_e4m3fn), self.recv_scale, self.recv_ids,
                                   self.recv_weights)
        returned = torch.empty((n_send + 1, self.hidden), dtype=torch.bfloat16, device=self.device)
        returned[n_send].zero_()                                           # row -1 of the gather below
        self._all_to_all(returned[:n_send], partial[:n_recv].contiguous(), send_split, recv_split)
        out = torch.zeros((tokens, self.hidden), dtype=torch.float32, device=self.device)
        for r in range(self.world):                                        # fixed rank order: deterministic sum
            out += returned[slot_of[:, r]].float()
        return out.to(torch.bfloat16)


def native_layer(weights: dict, *, capacity: int, experts: int, top_k: int = 8, act_mode: str = "fp8", device="cuda"):
    """(route, local_layer) built on the native kernels for one rank; ``weights`` holds the rank's
    gemm1/gemm2 weights and scales and ``local_expert_offset``."""
    from . import ops

    state = {}

    def route_factory(mode: str, n_group=8, topk_group=4):
        def route(logits, bias, factor):
            key = ("route", logits.data_ptr(), bias.data_ptr(), factor.data_ptr())
            if key not in state:
                t = logits.shape[0]
                ids = torch.empty((t, top_k), dtype=torch.int32, device=device)
                w = torch.empty((t, top_k), dtype=torch.float32, device=device)
                state[key] = (ops.MoeRouting(logits, bias, factor, ids, w, top_k=top_k, n_group=n_group,
                                             topk_group=topk_group, mode=mode), ids, w)
            op, ids, w = state[key]
            op.launch()
            return ids, w
        return route

    def local_layer(hidden, scale, ids, w):
        key = ("layer", hidden.data_ptr(), scale.data_ptr(), ids.data_ptr(), w.data_ptr())
        if key not in state:
            out = torch.empty((capacity, hidden.shape[1]), dtype=torch.bfloat16, device=device)
            inputs = dict(weights)
            inputs.update(expert_ids=ids, route_weights=w, hidden_states=hidden, hidden_states_scale=scale)
            state[key] = (ops.Fp8Moe(inputs, out, experts=experts, top_k=top_k, act_mode=act_mode, external_routing=True), out)
        op, out = state[key]
        op.launch()
        return out

    return route_factory, local_layer


class NativeExpertParallelMoe:
    """The same layer on the native exchange kernels (``cake_b200_ep_exchange_*``): every shape is
    static -- each rank exchanges ``tokens`` rows with every peer, unused rows carry expert id -1 --
    so a step is kernel launches and two equal-split all-to-alls with no host synchronisation.

    ``weights`` holds this rank's ``gemm1_weights``, ``gemm1_weights_scale``, ``gemm2_weights``,
    ``gemm2_weights_scale``, ``local_expert_offset`` and ``routed_scaling_factor``; the token inputs
    are bound at construction (their device buffers are reused every step)."""

    def __init__(self, weights: dict, routing_logits, routing_bias, hidden_states, hidden_states_scale, *,
                 experts: int, top_k: int = 8, routing: str = "softmax", n_group: int = 8, topk_group: int = 4,
                 act_mode: str = "fp8", group=None):
        import ctypes

        from . import _lib, ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        dev = hidden_states.device
        self.device = dev
        tokens, hidden = hidden_states.shape
        self.tokens, self.hidden, self.top_k = tokens, hidden, top_k
        cap = tokens
        rows = self.world * cap
        cfg = _lib.EpConfig(tokens, cap, hidden, top_k, self.world, experts)
        width = int(_lib.library().cake_b200_ep_row_bytes(ctypes.byref(cfg)))
        if width == 0:
            raise ValueError("unsupported expert-parallel configuration (hidden must be a multiple of 512 and top_k even)")
        i32, f32 = torch.int32, torch.float32
        self.ids = torch.empty((tokens, top_k), dtype=i32, device=dev)
        self.route_weights = torch.empty((tokens, top_k), dtype=f32, device=dev)
        self.slot_of = torch.empty((tokens, self.world), dtype=i32, device=dev)
        self.send = torch.zeros((self.world, cap, width), dtype=torch.uint8, device=dev)
        self.recv = torch.zeros((self.world, cap, width), dtype=torch.uint8, device=dev)
        self.recv_hidden = torch.zeros((rows, hidden), dtype=torch.float8_e4m3fn, device=dev)
        self.recv_scale = torch.zeros((hidden // 128, rows), dtype=f32, device=dev)
        self.recv_ids = torch.full((rows, top_k), -1, dtype=i32, device=dev)
        self.recv_weights = torch.zeros((rows, top_k), dtype=f32, device=dev)
        self.partial = torch.empty((rows, hidden), dtype=torch.bfloat16, device=dev)
        self.returned = torch.empty((self.world, cap, hidden), dtype=torch.bfloat16, device=dev)
        self.output = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.router = ops.MoeRouting(routing_logits, routing_bias, weights["routed_scaling_factor"], self.ids,
                                     self.route_weights, top_k=top_k, n_group=n_group, topk_group=topk_group, mode=routing)
        layer_inputs = dict(weights)
        layer_inputs.update(expert_ids=self.recv_ids, route_weights=self.recv_weights, hidden_states=self.recv_hidden,
                            hidden_states_scale=self.recv_scale)
        self.layer = ops.Fp8Moe(layer_inputs, self.partial, experts=experts, top_k=top_k, act_mode=act_mode,
                                external_routing=True)
        buffers = [self.ids, self.route_weights, hidden_states, hidden_states_scale, self.slot_of, self.send, self.recv,
                   self.recv_hidden, self.recv_scale, self.recv_ids, self.recv_weights, self.returned, self.output]
        self._keep = buffers
        pointers = (ctypes.c_void_p * len(buffers))(*[t.data_ptr() for t in buffers])
        self._handle = ctypes.c_void_p()
        with torch.cuda.device(dev):
            code = _lib.library().cake_b200_ep_exchange_create(pointers, ctypes.byref(cfg), ctypes.byref(self._handle))
        if code:
            raise _lib.CakeError("cake_b200_ep_exchange_create", code)
        self._lib = _lib
        # kernels of this library launched per step: routing 1, exchange 4, rank-local layer 7
        self.launches_per_step = 12

    def _stage(self, stage: int):
        code = self._lib.library().cake_b200_ep_exchange_launch_stage(self._handle, stage, torch.cuda.current_stream().cuda_stream)
        if code:
            raise self._lib.CakeError("cake_b200_ep_exchange_launch_stage", code)

    def capture(self) -> None:
        """Records one step (kernels and both all-to-alls) into a CUDA graph on a side stream; later
        ``forward()`` calls replay it, which removes the per-launch host cost that dominates once a rank's
        share of the layer is a few hundred microseconds.  Call after at least one eager step."""
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            self._eager()                       # settle lazy initialisation on this stream
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                self._eager()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self._graph = graph

    def forward(self) -> torch.Tensor:
        if getattr(self, "_graph", None) is not None:
            self._graph.replay()
            return self.output
        return self._eager()

    STEP_PARTS = ("route_plan_pack", "dispatch_all_to_all", "unpack", "layer_route_permute_gather", "layer_gemm1_swiglu",
                  "layer_gemm2", "layer_combine", "return_all_to_all", "reduce")

    def _parts(self):
        """The parts of one step, in order, as closures on the current stream."""
        def dispatch():
            if self.world == 1:
                self.recv.copy_(self.send)
            else:
                dist.all_to_all_single(self.recv, self.send, group=self.group)

        def give_back():
            if self.world == 1:
                self.returned.copy_(self.partial.view_as(self.returned))
            else:
                dist.all_to_all_single(self.returned, self.partial.view_as(self.returned), group=self.group)

        def route_plan_pack():
            self.router.launch()
            self._stage(0)

        return [route_plan_pack, dispatch, lambda: self._stage(1), lambda: self.layer.launch_stage(0),
                lambda: self.layer.launch_stage(1), lambda: self.layer.launch_stage(2), lambda: self.layer.launch_stage(3),
                give_back, lambda: self._stage(2)]

    def _eager(self) -> torch.Tensor:
        with torch.cuda.device(self.device):
            for part in self._parts():
                part()
        return self.output

    def stage_times(self, steps: int = 5) -> dict:
        """Mean milliseconds of each part of a step (STEP_PARTS), eager launches with an event after every part.
        A collective's time includes waiting for the slowest peer to arrive at it."""
        with torch.cuda.device(self.device):
            parts = self._parts()
            events = [[torch.cuda.Event(enable_timing=True) for _ in range(len(parts) + 1)] for _ in range(steps)]
            for k in range(steps):
                events[k][0].record()
                for i, part in enumerate(parts):
                    part()
                    events[k][i + 1].record()
            torch.cuda.synchronize(self.device)
        return {name: sum(events[k][i].elapsed_time(events[k][i + 1]) for k in range(steps)) / steps
                for i, name in enumerate(self.STEP_PARTS)}

    def close(self):
        if self._handle.value:
            self._lib.library().cake_b200_ep_exchange_destroy(self._handle)
            import ctypes
            self._handle = ctypes.c_void_p()


class PushExpertParallelMoe:
    """The expert-parallel layer with the exchange done by the ranks' own kernels over NVLink
    (``cake_b200_ep_push_*``): a rank writes each needed row straight into the receive block of the rank that owns
    the expert, and each partial row straight back into the token owner's block, inside one symmetric buffer per
    rank that ``torch.distributed._symmetric_memory`` maps into every peer.  No collective call is left in a step,
    only the needed rows travel, and the rank-local layer sees the received rows compacted.  A step is
    route -> plan + push -> wait + unpack -> layer stages 0..2 -> combine + push back -> wait + reduce, all on the
    caller's stream; ``capture()`` records it as one CUDA graph.  Same constructor as ``NativeExpertParallelMoe``.
    With a world of one the symmetric buffer is an ordinary tensor and the rank pushes to itself."""

    STEP_PARTS = ("route_plan_push", "wait_unpack", "layer_route_permute_gather", "layer_gemm1_swiglu", "layer_gemm2",
                  "combine_push_back", "wait_reduce")

    def __init__(self, weights: dict, routing_logits, routing_bias, hidden_states, hidden_states_scale, *,
                 experts: int, top_k: int = 8, routing: str = "softmax", n_group: int = 8, topk_group: int = 4,
                 act_mode: str = "fp8", group=None, virtual=None):
        """``virtual = (rank, world, buffers)`` makes this object one of ``world`` ranks that all live in this
        process on one GPU (``buffers``: one uint8 tensor of ``push_symmetric_bytes`` + 256 bytes per rank, zero-filled,
        shared by all of them), for tests that have fewer GPUs than ranks: the caller then runs the parts of a step
        (``_parts()``) in lock step, each part on every rank before the next, so that no kernel ever waits for a
        kernel that has not been launched."""
        import ctypes

        from . import _lib, ops
        self.group = group
        if virtual is not None:
            self.rank, self.world = int(virtual[0]), int(virtual[1])
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = hidden_states.device
        self.device = dev
        tokens, hidden = hidden_states.shape
        self.tokens, self.hidden, self.top_k = tokens, hidden, top_k
        cap = tokens
        rows = self.world * cap
        cfg = _lib.EpPushConfig(tokens, cap, hidden, top_k, self.world, experts, self.rank)
        lib = _lib.library()
        sym_bytes = int(lib.cake_b200_ep_push_symmetric_bytes(ctypes.byref(cfg)))
        if sym_bytes == 0:
            raise ValueError("unsupported expert-parallel configuration (hidden must be a multiple of 512 and top_k even)")
        i32, f32 = torch.int32, torch.float32
        with torch.cuda.device(dev):
            if virtual is not None:
                self.symmetric = virtual[2][self.rank]
                bases = [(b.data_ptr() + 255) // 256 * 256 for b in virtual[2]]
            elif self.world > 1:
                import torch.distributed._symmetric_memory as symm
                self.symmetric = symm.empty(sym_bytes, dtype=torch.uint8, device=dev)
                self.symmetric.zero_()
                torch.cuda.synchronize(dev)
                self._symm_handle = symm.rendezvous(self.symmetric, group=dist.group.WORLD if group is None else group)
                bases = [int(p) for p in self._symm_handle.buffer_ptrs]
            else:
                self.symmetric = torch.zeros(sym_bytes + 256, dtype=torch.uint8, device=dev)
                bases = [(self.symmetric.data_ptr() + 255) // 256 * 256]
            self.peer_bases = torch.tensor(bases, dtype=torch.int64, device=dev)
            self.scratch = torch.zeros(int(lib.cake_b200_ep_push_scratch_bytes(ctypes.byref(cfg))) + 256, dtype=torch.uint8, device=dev)
            self.scratch_ptr = (self.scratch.data_ptr() + 255) // 256 * 256
        self.ids = torch.empty((tokens, top_k), dtype=i32, device=dev)
        self.route_weights = torch.empty((tokens, top_k), dtype=f32, device=dev)
        self.recv_hidden = torch.zeros((rows, hidden), dtype=torch.float8_e4m3fn, device=dev)
        self.recv_scale = torch.zeros((hidden // 128, rows), dtype=f32, device=dev)
        self.recv_ids = torch.full((rows, top_k), -1, dtype=i32, device=dev)
        self.recv_weights = torch.zeros((rows, top_k), dtype=f32, device=dev)
        self.partial = torch.empty((rows, hidden), dtype=torch.bfloat16, device=dev)     # the layer's own output: unused (stage 3 is not run)
        self.output = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.router = ops.MoeRouting(routing_logits, routing_bias, weights["routed_scaling_factor"], self.ids,
                                     self.route_weights, top_k=top_k, n_group=n_group, topk_group=topk_group, mode=routing)
        layer_inputs = dict(weights)
        layer_inputs.update(expert_ids=self.recv_ids, route_weights=self.recv_weights, hidden_states=self.recv_hidden,
                            hidden_states_scale=self.recv_scale)
        self.layer = ops.Fp8Moe(layer_inputs, self.partial, experts=experts, top_k=top_k, act_mode=act_mode, external_routing=True)
        contributions, inv_perm = self.layer.intermediate("contributions"), self.layer.intermediate("inv_perm")
        own = bases[self.rank] if self.world > 1 else bases[0]
        pointers = [self.ids.data_ptr(), self.route_weights.data_ptr(), hidden_states.data_ptr(), hidden_states_scale.data_ptr(),
                    self.peer_bases.data_ptr(), own, self.scratch_ptr, self.recv_hidden.data_ptr(), self.recv_scale.data_ptr(),
                    self.recv_ids.data_ptr(), self.recv_weights.data_ptr(), contributions.data_ptr(), inv_perm.data_ptr(),
                    self.output.data_ptr()]
        self._keep = [hidden_states, hidden_states_scale, contributions, inv_perm]
        array = (ctypes.c_void_p * len(pointers))(*pointers)
        self._handle = ctypes.c_void_p()
        with torch.cuda.device(dev):
            code = lib.cake_b200_ep_push_create(array, ctypes.byref(cfg), ctypes.byref(self._handle))
        if code:
            raise _lib.CakeError("cake_b200_ep_push_create", code)
        self._lib = _lib
        if self.world > 1 and virtual is None:
            dist.barrier(group)            # every rank's buffers are zeroed and mapped before anyone pushes
        # kernels of this library launched per step: routing 1, exchange 6, rank-local layer stages 0..2: 6
        self.launches_per_step = 13
        self.slot_of = None

    def _stage(self, stage: int):
        code = self._lib.library().cake_b200_ep_push_launch_stage(self._handle, stage, torch.cuda.current_stream().cuda_stream)
        if code:
            raise self._lib.CakeError("cake_b200_ep_push_launch_stage", code)

    def _parts(self):
        def route_plan_push():
            self.router.launch()
            self._stage(0)
        return [route_plan_push, lambda: self._stage(1), lambda: self.layer.launch_stage(0), lambda: self.layer.launch_stage(1),
                lambda: self.layer.launch_stage(2), lambda: self._stage(2), lambda: self._stage(3)]

    def _eager(self) -> torch.Tensor:
        with torch.cuda.device(self.device):
            for part in self._parts():
                part()
        return self.output

    capture = NativeExpertParallelMoe.capture
    forward = NativeExpertParallelMoe.forward
    stage_times = NativeExpertParallelMoe.stage_times

    @staticmethod
    def symmetric_bytes(tokens: int, hidden: int, top_k: int, world: int, experts: int) -> int:
        """Bytes of one rank's symmetric buffer (``cake_b200_ep_push_symmetric_bytes``)."""
        import ctypes

        from . import _lib
        cfg = _lib.EpPushConfig(tokens, tokens, hidden, top_k, world, experts, 0)
        return int(_lib.library().cake_b200_ep_push_symmetric_bytes(ctypes.byref(cfg)))

    def status(self) -> int:
        """0, or 5 when a wait for another rank's rows ran out (synchronises the stream)."""
        with torch.cuda.device(self.device):
            return self._lib.read_status(self.scratch_ptr, torch.cuda.current_stream().cuda_stream)

    def rows_sent(self) -> int:
        words = self.scratch[self.scratch_ptr - self.scratch.data_ptr() + 256:][:4 * (8 + 64)].view(torch.int32)
        return int(words[8:8 + self.world].sum().item())

    def close(self):
        if self._handle.value:
            self._lib.library().cake_b200_ep_push_destroy(self._handle)
            import ctypes
            self._handle = ctypes.c_void_p()
