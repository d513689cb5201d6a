"""cuda_sm100 forward: tensor validation, buffer ownership and the C-ABI call.

The Python side plays the role of the reference's binding layer
(csrc/backends/sm90/bindings.cpp:12-59 validation and allocation of out/final;
actlize_la/_gdn_ppu10.py:37-56 / actlize_la/serving/gdn_core.py:86-125 workspace
ownership and the ctypes launch): it checks shapes, dtypes, contiguity, alignment and
device, allocates output, optional final state and the workspace, and issues one
``actlize_la_sm100_forward_prepared`` call on the caller's current stream.  Inputs are
never modified; nothing is normalised, activated or rescaled here.
"""
from __future__ import annotations

from ._library import load_library
from .sm100_policy import policy, selection_for

MATH_CONTRACT = "wy-splitbf16-state-bf16-out-sm100-v1"
_DIAGNOSTIC_IDS = {"simt": 0, "umma": 1, "simt-prepare+umma-walk": 2, "umma-prepare+simt-walk": 3,
                   "umma-seg2": 1 | (2 << 8), "umma-seg4": 1 | (4 << 8), "umma-seg8": 1 | (8 << 8), "umma-seg16": 1 | (16 << 8),
                   # parallel sub-segments of the walk (bits 16..19), alone and with sequence segments
                   "umma-par2": 1 | (2 << 16), "umma-par3": 1 | (3 << 16), "umma-par4": 1 | (4 << 16),
                   "umma-par8": 1 | (8 << 16), "umma-seg2-par2": 1 | (2 << 8) | (2 << 16),
                   "umma-seg2-par4": 1 | (2 << 8) | (4 << 16), "umma-seg4-par4": 1 | (4 << 8) | (4 << 16)}


def configuration_id(name):
    try:
        return _DIAGNOSTIC_IDS[name]
    except KeyError:
        raise ValueError(f"unknown SM100 configuration: {name!r}; choose {tuple(_DIAGNOSTIC_IDS)}") from None


def _validate(q, k, v, g, beta, initial_state):
    import torch
    if q.ndim != 4 or v.ndim != 4 or k.shape != q.shape:
        raise ValueError("q/k must be [B,T,Hk,128] and v [B,T,Hv,128]")
    b, t, hk, d = q.shape
    hv = v.shape[2]
    if d != 128 or v.shape[3] != 128 or tuple(v.shape[:2]) != (b, t):
        raise ValueError("SM100 requires K=V=128 and matching batch/sequence")
    if min(b, t, hk, hv) < 1 or hv % hk:
        raise ValueError("SM100 requires positive sizes and Hv % Hk == 0")
    if tuple(g.shape) != (b, t, hv) or tuple(beta.shape) != (b, t, hv):
        raise ValueError("g and beta must be [B,T,Hv]")
    bf16, fp32 = torch.bfloat16, torch.float32
    if q.dtype != bf16 or k.dtype != bf16 or v.dtype != bf16 or beta.dtype != bf16:
        raise ValueError("q, k, v and beta must be BF16")
    if g.dtype not in (bf16, fp32):
        raise ValueError("g must be BF16/FP32 natural-log decay, not raw logits")
    tensors = [q, k, v, g, beta]
    if initial_state is not None:
        if tuple(initial_state.shape) != (b, hv, 128, 128) or initial_state.dtype != fp32:
            raise ValueError("initial_state must be FP32 [B,Hv,128,128] in K-by-V order")
        tensors.append(initial_state)
    for x in tensors:
        if x.device.type != "cuda" or x.device != q.device:
            raise ValueError("all tensors must be on the same CUDA device")
        if not x.is_contiguous():
            raise ValueError("all tensors must be contiguous")
        if x.requires_grad:
            raise ValueError("forward-only operator: inputs must not require grad")
    for x in (q, k, v):
        if x.data_ptr() % 16:
            raise ValueError("q, k and v must be 16-byte aligned")
    return b, t, hk, hv


class Sm100Forward:
    """A verified native library bound to the forward contract; identity checked once."""

    def __init__(self, library):
        self.library = library

    def workspace_bytes(self, b, t, hk, hv, config):
        n = self.library.lib.actlize_la_sm100_workspace_bytes(b, t, hk, hv, config)
        if n < 0:
            raise ValueError("geometry exceeds the native grid limits")
        return n

    def _workspace(self, device, nbytes):
        """Scratch of one call: a buffer kept per (device, current stream), grown on demand.  Calls on one stream
        follow each other in stream order, so they can share it; calls on different streams never do.  (The
        reference allocates its workspace per call from the caching allocator, actlize_la/_gdn_ppu10.py:48-55; with
        the host running several calls ahead of the device that keeps one workspace of hundreds of megabytes alive
        per call in flight, and the allocator's occasional cudaMalloc of one more stalls the host for milliseconds.)
        Under stream capture the buffer comes from the graph's own pool.  A configuration with several sequence
        segments additionally uses the library's per-device streams and events: only one such call may be in
        flight per device."""
        return self._stream_workspace(device, nbytes)

    def _side_stream(self, device):
        """One extra, high-priority stream per device for the state exchange (and the fold behind it) that runs next
        to the long output walk."""
        import torch
        streams = self.__dict__.setdefault("_side_streams", {})
        key = str(device)
        if key not in streams:
            streams[key] = torch.cuda.Stream(device=device, priority=-1)
        return streams[key]

    def _scratch_output(self, like):
        """A throw-away output buffer for the passes that produce states only, kept per device and shape (garbage
        by definition, so sharing it between calls is harmless)."""
        import torch
        cache = self.__dict__.setdefault("_scratch_cache", {})
        key = (like.device, tuple(like.shape))
        held = cache.get(key)
        if held is None:
            held = cache[key] = torch.empty_like(like)
            if len(cache) > 8:
                cache.pop(next(iter(cache)))
        return held

    def check_device_status(self, device=None, synchronize=True):
        """Raise RuntimeError if a kernel launched on ``device`` gave up a bounded wait.  Every wait inside the
        kernels is bounded; a kernel that runs out records where, drains and returns, and its output rows and
        final state are incomplete.  The forward itself never synchronises, so callers decide when to look: after
        their own synchronisation point (``synchronize=False``) or here (``synchronize=True``).  Each forward
        call also looks at the record first and raises for an earlier launch that failed."""
        import torch
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.library.configure(device)
        self.library.raise_on_failure(device, synchronize)

    def __call__(self, q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                 configuration=None, mode="device", sm_count=None):
        import torch
        b, t, hk, hv = _validate(q, k, v, g, beta, initial_state)
        if configuration is None:
            config = selection_for(q, v, mode=mode, sm_count=sm_count).configuration_id
        else:
            config = configuration_id(configuration)
        self.library.configure(q.device)
        self.library.raise_on_failure(q.device)        # an earlier launch that gave up: host-visible record, no sync
        out = torch.empty_like(v)
        final = (torch.empty((b, hv, 128, 128), dtype=torch.float32, device=q.device)
                 if output_final_state else None)
        nbytes = self.workspace_bytes(b, t, hk, hv, config)
        workspace = self._workspace(q.device, nbytes)
        if q.device.index != torch.cuda.current_device():
            with torch.cuda.device(q.device):
                return self._launch(q, k, v, g, beta, initial_state, out, final, workspace, nbytes, b, t, hk, hv, config)
        return self._launch(q, k, v, g, beta, initial_state, out, final, workspace, nbytes, b, t, hk, hv, config)

    def _launch(self, q, k, v, g, beta, initial_state, out, final, workspace, nbytes, b, t, hk, hv, config):
        import torch
        self.library.check(self.library.lib.actlize_la_sm100_forward_prepared(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
            initial_state.data_ptr() if initial_state is not None else None,
            out.data_ptr(), final.data_ptr() if final is not None else None,
            workspace.data_ptr(), nbytes, b, t, hk, hv,
            int(g.dtype == torch.float32), config, self.library.current_stream_handle(torch.cuda.current_device())))
        return out, final

    def prepare_segment(self, q, k, v, g, beta, reuse_workspace=False):
        """Run the prepare stage once and return a handle on which several walks can follow.  With
        ``reuse_workspace`` the factors go into a workspace kept per (device, current stream) instead of one
        allocated for this segment: for a caller that finishes with a segment before it prepares the next one on
        the same stream (stream order then keeps the two apart), so that a loop of calls whose host side runs ahead
        of the device does not hold, and allocate, one workspace of hundreds of megabytes per call in flight."""
        return PreparedSegment(self, q, k, v, g, beta, reuse_workspace)

    def _stream_workspace(self, device, nbytes):
        import torch
        if torch.cuda.is_current_stream_capturing():          # a graph keeps its own memory
            return torch.empty(nbytes, dtype=torch.uint8, device=device)
        cache = self.__dict__.setdefault("_stream_workspaces", {})
        index = device.index if device.index is not None else torch.cuda.current_device()
        key = (index, self.library.current_stream_handle(index))
        held = cache.get(key)
        if held is None or held.numel() < nbytes:
            cache.pop(key, None)
            while len(cache) >= 2:                            # these are large: keep the two most recent streams
                cache.pop(next(iter(cache)))
            held = cache[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return held

    def varlen(self, q, k, v, g, beta, cu_seqlens, initial_states=None, output_final_state=True):
        """Packed sequences in one prepare and one walk launch (actlize_la_sm100_forward_varlen)."""
        import ctypes
        import torch
        b, total, hk, hv = _validate(q, k, v, g, beta, None)
        on_device = isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda
        if on_device:
            # offsets that live on the device are handed over as they are: no host read, capturable
            if (cu_seqlens.dtype != torch.int32 or cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2
                    or cu_seqlens.device != q.device or not cu_seqlens.is_contiguous()):
                raise ValueError("device cu_seqlens must be a contiguous int32 vector [N+1] on the inputs' device")
            n, bounds = cu_seqlens.numel() - 1, None
            if b != 1:
                raise ValueError("varlen expects batch 1")
        else:
            bounds = [int(x) for x in cu_seqlens]
            n = len(bounds) - 1
            if b != 1 or n < 1 or bounds[0] != 0 or bounds[-1] != total:
                raise ValueError("varlen expects batch 1 and cu_seqlens running from 0 to the token count")
            if any(b1 < b0 for b0, b1 in zip(bounds, bounds[1:])):
                raise ValueError("cu_seqlens must be non-decreasing")
        if initial_states is not None:
            if (tuple(initial_states.shape) != (n, hv, 128, 128) or initial_states.dtype != torch.float32
                    or initial_states.device != q.device or not initial_states.is_contiguous()):
                raise ValueError("initial_states must be contiguous FP32 [N,Hv,128,128] on the inputs' device")
        self.library.configure(q.device)
        out = torch.empty_like(v)
        final = (torch.empty((n, hv, 128, 128), dtype=torch.float32, device=q.device)
                 if output_final_state else None)
        lib = self.library.lib
        nbytes = lib.actlize_la_sm100_varlen_workspace_bytes(total, n, hk, hv)
        if nbytes < 0:
            raise ValueError("geometry exceeds the native grid limits")
        workspace = self._workspace(q.device, nbytes)
        if on_device:
            with torch.cuda.device(q.device):
                self.library.check(lib.actlize_la_sm100_forward_varlen_device(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                    initial_states.data_ptr() if initial_states is not None else None,
                    out.data_ptr(), final.data_ptr() if final is not None else None,
                    workspace.data_ptr(), nbytes, cu_seqlens.data_ptr(), n, total, hk, hv,
                    int(g.dtype == torch.float32), torch.cuda.current_stream().cuda_stream))
            return out, final
        offsets = (ctypes.c_int * (n + 1))(*bounds)
        with torch.cuda.device(q.device):
            stream = torch.cuda.current_stream().cuda_stream
            self.library.check(lib.actlize_la_sm100_forward_varlen(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                initial_states.data_ptr() if initial_states is not None else None,
                out.data_ptr(), final.data_ptr() if final is not None else None,
                workspace.data_ptr(), nbytes, offsets, n, hk, hv, int(g.dtype == torch.float32), stream))
        return out, final


class PreparedSegment:
    """The WY factors of one token segment in a workspace of its own, and the walks over them.

    Used by the sequence-parallel scheme: the factors do not depend on the recurrent state, so the offset pass
    (zero state, only the deciding suffix), the transition pass (identity state, U treated as zero), the output walk
    and the correction pass (true incoming state) share the prepare work.  Built on stage-restricted calls of ``actlize_la_sm100_forward_prepared`` (tcgen05
    configuration); nothing is launched before the first method call.
    """
    _CONFIG, _PREPARE, _WALK, _HOMOGENEOUS, _UNTIL_DECAYED, _OFFSET_TAIL, _PAIR = 1, 0x10, 0x20, 0x40, 0x80, 0x100000, 0x200000

    def __init__(self, owner, q, k, v, g, beta, reuse_workspace=False):
        import torch
        self.dims = _validate(q, k, v, g, beta, None)
        self.owner, self.tensors = owner, (q, k, v, g, beta)
        b, t, hk, hv = self.dims
        owner.library.configure(q.device)
        selection = selection_for(q, v)
        # the walk alone, split into the policy's parallel sub-segments
        self.split_walk = self._CONFIG | self._WALK | ((selection.parallel << 16) if selection.parallel > 1 else 0)
        self.nbytes = owner.workspace_bytes(b, t, hk, hv, self._CONFIG)
        self.workspace = (owner._stream_workspace(q.device, self.nbytes) if reuse_workspace
                          else torch.empty(self.nbytes, dtype=torch.uint8, device=q.device))
        self.output = torch.empty_like(v)
        self._side = self.pair = None
        # what every launch passes, looked up once
        self._entry = owner.library.lib.actlize_la_sm100_forward_prepared
        self._pointers = tuple(x.data_ptr() for x in self.tensors)
        self._workspace_pointer = self.workspace.data_ptr()
        self._gate_fp32 = int(g.dtype == torch.float32)
        self._device_index = q.device.index if q.device.index is not None else torch.cuda.current_device()

    def _launch(self, config, initial, output, final):
        import torch
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self._device_index):
                return self._launch(config, initial, output, final)
        b, t, hk, hv = self.dims
        self.owner.library.check(self._entry(
            *self._pointers, initial.data_ptr() if initial is not None else None, output.data_ptr(),
            final.data_ptr() if final is not None else None, self._workspace_pointer, self.nbytes,
            b, t, hk, hv, self._gate_fp32, config, self.owner.library.current_stream_handle(self._device_index)))

    def _state(self):
        import torch
        b, _, _, hv = self.dims
        return torch.empty((b, hv, 128, 128), dtype=torch.float32, device=self.output.device)

    def early_pair(self, need_transition=True):
        """(b_r, M_r) of ``S_out = M_r S_in + b_r``, produced EARLY: the prepare launch, then ONE short launch on the
        same stream that holds, per (batch, value head), the offset pass (only the suffix of the segment that
        decides the outgoing state, from zero: a few chunks when the gate decays) and, if asked for, the transition
        pass (exact zeros at once for a head whose segment decays below exp(-40)).  The caller launches the long
        output walk next (``walk_outputs``) and exchanges the pair inside ``side()``, a second stream that starts
        behind the short launch, while that walk runs; ``join()`` orders the current stream behind the side stream."""
        import torch
        self._launch(self._CONFIG | self._PREPARE, None, self.output, None)
        scratch = self.owner._scratch_output(self.output)
        if need_transition:
            # the pair in one block [2, B, Hv, 128, 128] = (M_r, b_r): it travels as one message
            b, _, _, hv = self.dims
            self.pair = torch.empty((2, b, hv, 128, 128), dtype=torch.float32, device=self.output.device)
            self._launch(self._CONFIG | self._WALK | self._PAIR, None, scratch, self.pair)
            offset, transition = self.pair[1], self.pair[0]
        else:
            self.pair = None
            offset, transition = self._state(), None
            self._launch(self._CONFIG | self._WALK | self._OFFSET_TAIL, None, scratch, offset)
        if self._side is None:
            self._side = self.owner._side_stream(self.output.device)
        self._side.wait_stream(torch.cuda.current_stream())
        (self.pair if need_transition else offset).record_stream(self._side)
        return offset, transition

    def walk_outputs(self, initial=None):
        """The output rows of the segment walked from ``initial`` (zero when None) over the prepared factors, split
        into the policy's parallel sub-segments; no final state (``early_pair`` has the outgoing state)."""
        self._launch(self.split_walk, initial, self.output, None)
        return self.output

    def side(self):
        """Context manager: work issued inside runs on the side stream, behind the passes of ``early_pair``."""
        import torch
        return torch.cuda.stream(self._side)

    def join(self, *tensors):
        """The current stream waits for the side stream; ``tensors`` made there may then be used on it."""
        import torch
        current = torch.cuda.current_stream()
        current.wait_stream(self._side)
        for x in tensors:
            if x is not None:
                x.record_stream(current)

    def prepare(self):
        """Only the factors (for a rank that has nothing else to do before its incoming state arrives)."""
        self._launch(self._CONFIG | self._PREPARE, None, self.output, None)

    def finish(self, incoming, output_final_state=True):
        """The ordinary walk from the true incoming state over prepared factors: (output, final state or None)."""
        final = self._state() if output_final_state else None
        self._launch(self._CONFIG | self._WALK, incoming, self.output, final)
        return self.output, final

    def finish_decayed(self, incoming):
        """Rewrite only the leading chunks of ``self.output`` (those the incoming state still reaches, decay
        above exp(-40) per batch and value head); valid after ``walk_outputs(None)`` has written the zero-state rows."""
        self._launch(self._CONFIG | self._WALK | self._UNTIL_DECAYED, incoming, self.output, None)
        return self.output


_FORWARD = {}


def load_sm100():
    """The forward bound to the verified native library; no kernel is launched by loading."""
    library = load_library()
    forward = _FORWARD.get(id(library))
    if forward is None:
        forward = _FORWARD[id(library)] = Sm100Forward(library)
    return forward


def gdn_chunk_sm100(q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                    backend="cuda_sm100", configuration=None, mode="device", sm_count=None):
    """Explicit complete cuda_sm100 algorithm (the `wy_sm100` catalog entry)."""
    if backend != "cuda_sm100":
        raise ValueError(f"wy_sm100 cannot execute on {backend}")
    if configuration is not None and configuration not in _DIAGNOSTIC_IDS:
        raise ValueError(f"unknown SM100 configuration: {configuration}")
    return load_sm100()(q, k, v, g, beta, initial_state, output_final_state,
                        configuration=configuration, mode=mode, sm_count=sm_count)


def registered_configurations():
    return tuple(policy()["configurations"])
