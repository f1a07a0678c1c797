"""Token loops around the megakernel.

Reference: megakernels/generators.py (``Generator.generate_with_eos`` :21-58,
``MK_Generator`` :95-163).  The per-token host contract is unchanged: write the
token embedding into ``globs.hidden_states``, zero the barriers, set
``pos_id``, launch, read ``argmax(globs.logits)``.  Everything stays on the
device and nothing synchronises inside the loop.
"""

from __future__ import annotations

import torch
from torch import Tensor

from megakernels_b200.mk import MK_Interpreter
from megakernels_b200.model_types import BatchState
from megakernels_b200.scheduler import Schedule


class Generator:
    def generate(
        self,
        output_tokens: Tensor,
        prompt_len: int,
        ntok: int,
        ntok_already_generated: int = 1,
    ):
        raise NotImplementedError

    def generate_with_eos(
        self,
        output_tokens: Tensor,
        prompt_len: int,
        ntok: int,
        eos_token_check_interval: int,
        eos_token_ids: list[int],
    ):
        """Generate in chunks, stopping at the first EOS token.

        Returns ``(position of the first eos, number of tokens generated)``
        (reference: megakernels/generators.py:21-58).
        """
        assert output_tokens.shape[0] == 1, "batch size must be 1"
        eos = set(int(t) for t in eos_token_ids)
        for done in range(1, ntok, eos_token_check_interval):
            chunk = min(eos_token_check_interval, ntok - done)
            self.generate(
                output_tokens, prompt_len=prompt_len, ntok=chunk, ntok_already_generated=done
            )
            new = output_tokens[0, done : done + chunk].cpu().tolist()
            for j, tok in enumerate(new):
                if tok in eos:
                    return done + j, done + chunk - 1
        return ntok, ntok - 1


class MK_Generator(Generator):
    """Greedy decoding, one megakernel launch per token.

    As in the reference one sequence (``generate``, ``prefill``).  With a schedule built
    for ``LatencyScheduleOptions(batch_size=B)`` the same ``run`` advances B independent
    sequences by one token per launch: ``input_ids`` is ``[B, 1]``, ``pos_id`` a list of B
    positions (sequence b lives in slot b of the KV cache), the result ``[B]`` token ids.
    """

    def __init__(
        self,
        model,
        interpreter: MK_Interpreter,
        schedule: Schedule,
        barrier_fill_val: int = 0,
        skip_mk: bool = False,
        skip_rest: bool = False,
        fused_argmax: bool = True,
    ):
        self.model = model
        self.interpreter = interpreter
        self.schedule = schedule
        self.barrier_fill_val = barrier_fill_val
        self.skip_mk = skip_mk
        self.skip_rest = skip_rest
        self.last_call = None
        self.fill()
        # The kernel's LM-head epilogue can deliver argmax(logits) itself (the reference runs
        # torch.argmax over the 128k logits after the kernel, generators.py:143).  Only for
        # schedules that contain the LM head and when the megakernel actually runs.
        globs = schedule.globs
        has_head = globs.instructions is not None and bool((globs.instructions[:, :, 0] == 7).any())
        # (the tcgen05 build for more than 8 sequences leaves the argmax to the host)
        if fused_argmax and has_head and not skip_mk and globs.hidden_states.is_cuda and globs.batch_size <= 8:
            globs.argmax_out = torch.zeros(
                globs.batch_size, dtype=torch.int32, device=globs.hidden_states.device
            )

    def fill(self):
        """Reset the per-token VM state: barrier counters and residual accumulators."""
        globs = self.schedule.globs
        if self.barrier_fill_val == 0 and globs.vm_state is not None:
            globs.vm_state.zero_()  # one buffer behind both
            return
        globs.barriers.fill_(self.barrier_fill_val)
        if globs.residual_acc is not None:
            globs.residual_acc.zero_()

    def replace_with_noops(self):
        self.schedule.globs.instructions.zero_()

    # -- CUDA-graph replay of one decode step -------------------------------- #
    def enable_cuda_graph(self, warmup_pos: int = 0):
        """Capture one decode step (embed, barrier reset, kernel launches, collectives,
        argmax) into a CUDA graph that every later ``run`` replays.

        The position is then read by the kernel from a device word
        (``globs.pos_id_device``) and the input token from a device buffer, so one
        graph serves all tokens and the per-launch host work disappears.  The
        reference launches eagerly (megakernels/generators.py:121-143).
        """
        globs = self.schedule.globs
        device = globs.hidden_states.device
        B = globs.batch_size
        self._graph_tok = torch.zeros(B, 1, dtype=torch.long, device=device)
        self._graph_out = torch.zeros(B, dtype=torch.long, device=device)
        globs.pos_id_device = torch.full((B,), warmup_pos, dtype=torch.int32, device=device)
        globs.pos_id = warmup_pos
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(2):  # first calls allocate (status record, descriptor cache, NCCL)
                self._graph_out.copy_(self._step(self._graph_tok).reshape(-1))
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._graph_out.copy_(self._step(self._graph_tok).reshape(-1))
        return self

    def _step(self, input_ids: Tensor) -> Tensor:
        """The device work of one token; the position is already in the globals."""
        globs = self.schedule.globs
        post = self.model.model.embed_tokens(BatchState(input_ids=input_ids))
        globs.hidden_states[:] = post.hidden_states.reshape(globs.hidden_states.shape)
        self.fill()
        self.last_call = self.interpreter.interpret(globs)
        return self._next_token()

    def _next_token(self) -> Tensor:
        globs = self.schedule.globs
        if globs.argmax_out is not None:
            return globs.argmax_out.to(torch.long)
        return torch.argmax(globs.logits, dim=-1)

    def _replay(self, input_ids: Tensor, pos_id) -> Tensor:
        self._graph_tok.copy_(input_ids.reshape(self._graph_tok.shape))
        if isinstance(pos_id, int):
            self.schedule.globs.pos_id_device.fill_(pos_id)
        else:  # one position per sequence
            self.schedule.globs.pos_id_device.copy_(torch.as_tensor(pos_id, dtype=torch.int32), non_blocking=True)
        self._graph.replay()
        return self._graph_out

    def run(self, input_ids: Tensor, pos_id):
        if getattr(self, "_graph", None) is not None:
            return self._replay(input_ids, pos_id)
        globs = self.schedule.globs
        if not self.skip_rest:
            post = self.model.model.embed_tokens(BatchState(input_ids=input_ids))
            assert post.hidden_states is not None
            globs.hidden_states[:] = post.hidden_states.reshape(globs.hidden_states.shape)
        self.fill()
        if globs.batch_size > 1:
            globs.pos_ids = [int(p) for p in pos_id]
            assert len(globs.pos_ids) == globs.batch_size
            if globs.batch_size > 8:  # more positions than the launch struct holds: device array
                if globs.pos_id_device is None:
                    globs.pos_id_device = torch.zeros(
                        globs.batch_size, dtype=torch.int32, device=globs.hidden_states.device
                    )
                globs.pos_id_device.copy_(torch.tensor(globs.pos_ids, dtype=torch.int32), non_blocking=True)
        else:
            globs.pos_id = pos_id
        if not self.skip_mk:
            self.last_call = self.interpreter.interpret(globs)
        if self.skip_rest:
            return input_ids
        return self._next_token()

    def generate(
        self,
        output_tokens: Tensor,
        prompt_len: int,
        ntok: int,
        ntok_already_generated: int = 1,
    ):
        """Fill ``output_tokens[:, already : already + ntok]`` greedily.

        ``pos_id = prompt_len + ntok_already_generated + i - 1``
        (reference: megakernels/generators.py:145-163).
        """
        for i in range(ntok):
            in_pos = ntok_already_generated + i - 1
            input_ids = output_tokens[:, in_pos : in_pos + 1]
            pos_id = prompt_len + ntok_already_generated + i - 1
            output_ids = self.run(input_ids, pos_id=pos_id)
            output_tokens[:, in_pos + 1] = output_ids.reshape(-1)

    def prefill(self, prompt_ids: Tensor) -> Tensor:
        """Run the prompt through the decode kernel one token at a time.

        The reference prefills with its torch model (scripts/generate.py:125-137);
        here the KV cache is filled by the megakernel itself, so no second
        implementation of the forward pass exists in the product.  Returns the
        first generated token ``[1]``.
        """
        ids = prompt_ids.reshape(1, -1)
        out = None
        for pos in range(ids.shape[1]):
            out = self.run(ids[:, pos : pos + 1], pos_id=pos)
        return out.reshape(-1)

    def check(self):
        """Synchronise and raise if any device-side wait gave up."""
        if self.last_call is None:
            return None
        import mk_llama  # the module get_mk_func imported

        return mk_llama.sync_status(self.last_call)


class TP_MK_Generator(MK_Generator):
    """Megatron-style tensor-parallel decoding, one rank per GPU.

    The reference's kernel has no tensor parallelism; its torch model shards
    q/k/v/up/gate by rows and o/down by columns (megakernels/llama.py:665-691).
    Here every rank runs the megakernel on its shard (``model`` built with
    ``ExtraModelConfig(tp_size, tp_rank)``).  The instruction stream is cut after
    every o-proj and down-proj group; between two cuts the ranks all-reduce the
    residual accumulators (``globs.residual_acc``, 64-bit fixed point).  Each rank
    adds ``tp_size`` times its partial projection to its full copy
    (``globs.residual_scale``), so that the sum over ranks divided by ``tp_size``
    - an exact integer division - equals ``previous value + sum of partials`` on
    every rank, bit for bit, and nothing has to be zeroed between segments.
    """

    def __init__(self, model, interpreter, schedule, group=None, sched: str = "rr", all_reduce=None):
        from megakernels_b200.demos.latency.scheduler import split_at_collectives
        from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

        super().__init__(model, interpreter, schedule)
        self.group = group
        self.tp_size = model.extra_config.tp_size
        globs = schedule.globs
        globs.residual_scale = float(self.tp_size)
        self.segments = []
        for instructions, needs_all_reduce in split_at_collectives(schedule.get_linear_instructions()):
            queues = assign_to_sms(sched, instructions=instructions, sm_count=globs.sm_count())
            tensorize_instructions(globs, queues)
            self.segments.append((globs.instructions, globs.timings, needs_all_reduce))
        self.all_reduce = all_reduce or self._nccl_average

    def _nccl_average(self, tensor: Tensor):
        import torch.distributed as dist

        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        tensor.floor_divide_(self.tp_size)  # every term is a multiple of tp_size: exact

    def begin_token(self, input_ids: Tensor, pos_id: int):
        globs = self.schedule.globs
        post = self.model.model.embed_tokens(BatchState(input_ids=input_ids))
        globs.hidden_states[:] = post.hidden_states.reshape(-1)
        self.fill()
        globs.pos_id = pos_id

    def launch_segment(self, k: int) -> bool:
        """Enqueue segment ``k``; returns whether an all-reduce must follow it."""
        globs = self.schedule.globs
        globs.instructions, globs.timings, needs_all_reduce = self.segments[k]
        self.last_call = self.interpreter.interpret(globs)
        return needs_all_reduce

    def finish_token(self) -> Tensor:
        return torch.argmax(self.schedule.globs.logits, dim=-1)

    def _step(self, input_ids: Tensor) -> Tensor:
        globs = self.schedule.globs
        post = self.model.model.embed_tokens(BatchState(input_ids=input_ids))
        globs.hidden_states[:] = post.hidden_states.reshape(-1)
        self.fill()
        for k in range(len(self.segments)):
            if self.launch_segment(k):
                self.all_reduce(globs.residual_acc)
        return self.finish_token()

    def run(self, input_ids: Tensor, pos_id: int):
        if getattr(self, "_graph", None) is not None:
            return self._replay(input_ids, pos_id)
        self.schedule.globs.pos_id = pos_id
        return self._step(input_ids)


class TP_Peer_MK_Generator(MK_Generator):
    """Tensor-parallel decoding with the all-reduce inside the kernel: one launch per token.

    No counterpart in the reference.  The schedule must have been built with
    ``LatencyScheduleOptions(tp_all_reduce_chunks=n)`` on a model shard
    (``ExtraModelConfig(tp_size, tp_rank)``), which puts ``TP_AllReduce``
    instructions after every o-proj and down-proj group; this class attaches the
    peer-mapped buffers (``megakernels_b200.peer.connect``, a collective over
    ``group``) and keeps the launch counter from which the device derives the tag
    of every exchanged value.  All ranks must call ``run`` the same number of
    times; the ranks' kernels wait for each other with a time budget, so a rank
    that stops shows up as ``MegakernelError`` (device timeout) on the others.

    Recovery rule (include/mkb200.h, MkbTensorParallel): a launch that was aborted
    has already stored partial sums carrying the current launch counter's tags.
    Before the next launch every rank must therefore move to a counter value no
    rank has used yet: ``check`` (a collective) does that whenever any rank
    reports an error, ``resync_epoch`` does it unconditionally.
    """

    def __init__(self, model, interpreter, schedule, group=None):
        from megakernels_b200 import peer

        super().__init__(model, interpreter, schedule)
        self.group = group
        self.block = peer.connect(schedule.globs, group)

    def _step(self, input_ids: Tensor) -> Tensor:
        out = super()._step(input_ids)
        tp = self.schedule.globs.tp
        tp.epoch_device.add_(1)  # on the launch stream: the next launch reads the new value
        return out

    def run(self, input_ids: Tensor, pos_id: int):
        if getattr(self, "_graph", None) is not None:
            return self._replay(input_ids, pos_id)  # the captured step includes the increment
        self.schedule.globs.pos_id = pos_id
        return self._step(input_ids)

    def resync_epoch(self) -> int:
        """Collective: set every rank's launch counter to (max over ranks) + 1.

        Tags of an aborted launch can then never match again, whatever subset of
        the ranks took part in it.  Returns the new value.
        """
        import torch.distributed as dist

        tp = self.schedule.globs.tp
        top = tp.epoch_device.clone()
        dist.all_reduce(top, op=dist.ReduceOp.MAX, group=self.group)
        tp.epoch_device.copy_(top + 1)
        return int(tp.epoch_device)

    def check(self):
        """Collective status check: synchronise, learn whether ANY rank's launch gave up,
        and if so resynchronise the launch counters before raising.

        Raises the rank's own ``MegakernelError``, or ``RuntimeError`` on ranks whose
        launch ran clean while a peer's did not.
        """
        import torch.distributed as dist

        import mk_llama

        err = None
        try:
            status = super().check()
        except mk_llama.MegakernelError as e:
            status, err = None, e
        device = self.schedule.globs.hidden_states.device
        failed = torch.tensor([1 if err is not None else 0], dtype=torch.int32, device=device)
        dist.all_reduce(failed, op=dist.ReduceOp.MAX, group=self.group)
        if int(failed):
            self.resync_epoch()
            if err is not None:
                raise err
            raise RuntimeError("a tensor-parallel peer reported a device error; launch counters resynchronised")
        return status

    def close(self):
        self._graph = None
        self.block.close()
