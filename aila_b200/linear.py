"""Host-side mirror of the reference operator ``Bnb4BitLinear`` over the C-ABI library.

Names, argument meaning and error behaviour follow reference src/ops/Bnb4BitLinear.hpp:12-59:
``init`` / ``init_fused_rows`` return ``False`` and set ``last_error`` on invalid input,
``forward`` raises ``RuntimeError`` for a non-bf16 tensor or ``seq_len <= 0``
(Bnb4BitLinear.cpp:805-811), ``try_forward_decode_gate_up_swiglu`` returns ``False`` when the
fused path does not apply (:764-776). torch supplies device memory and streams only.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .synth import Nf4Tensors


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


class Bnb4BitLinearScratch:
    """Per-engine work space (reference Bnb4BitLinearScratch, Bnb4BitLinear.hpp:12-24)."""

    def __init__(self, device: int | torch.device = 0):
        self.device = torch.device("cuda", device) if isinstance(device, int) else device
        lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(lib.aila_nf4_scratch_create(self.device.index or 0, ctypes.byref(h)))
        self._h = h

    def ensure(self, seq_len: int, in_features: int, out_features: int, need_weight: bool) -> None:
        """Bnb4BitLinearScratch::ensure (Bnb4BitLinear.cpp:414-451): grow-only pre-sizing."""
        _lib.check(_lib.load().aila_nf4_scratch_reserve(self._h, seq_len, in_features, out_features,
                                                        1 if need_weight else 0))

    def check(self) -> None:
        """Raises if a bounded wait inside a kernel expired since the last check."""
        _lib.check(_lib.load().aila_nf4_scratch_check(self._h, _stream_ptr(self.device)))

    def set_wait_limit(self, sm_cycles: int) -> None:
        """Bound (SM clock cycles) of every device-side wait of the chained decode kernel."""
        _lib.check(_lib.load().aila_nf4_scratch_set_wait_limit(self._h, int(sm_cycles)))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.load().aila_nf4_scratch_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _np_ptr(a: np.ndarray | None) -> int | None:
    return None if a is None else a.ctypes.data


class Bnb4BitLinear:
    """One NF4 linear on one GPU (reference class Bnb4BitLinear, Bnb4BitLinear.hpp:26-59)."""

    def __init__(self):
        self._h = None
        self.last_error = ""
        self.device = None

    # -- construction -----------------------------------------------------------------
    @staticmethod
    def _desc(w: Nf4Tensors, device: int, keep: list) -> _lib.WeightDesc:
        d = _lib.WeightDesc()
        d.out_features, d.in_features, d.blocksize = w.out_features, w.in_features, w.blocksize
        d.nested = 1 if w.nested else 0
        d.nested_blocksize = w.nested_blocksize if w.nested else 0
        d.nested_offset = float(w.nested_offset) if w.nested else 0.0
        packed = np.ascontiguousarray(w.packed, np.uint8)
        absmax = np.ascontiguousarray(w.absmax_codes, np.uint8) if w.nested else \
            np.ascontiguousarray(w.absmax_f32, np.float32)
        qmap = np.ascontiguousarray(w.quant_map, np.float32)
        keep += [packed, absmax, qmap]
        d.packed_weight, d.absmax, d.quant_map = packed.ctypes.data, absmax.ctypes.data, qmap.ctypes.data
        if w.nested:
            nabs = np.ascontiguousarray(w.nested_absmax, np.float32)
            nmap = np.ascontiguousarray(w.nested_quant_map, np.float32)
            keep += [nabs, nmap]
            d.nested_absmax, d.nested_quant_map = nabs.ctypes.data, nmap.ctypes.data
            d.nested_absmax_count = nabs.size
        d.pointers_on_device = 0
        d.device = device
        return d

    def init(self, weight: Nf4Tensors, device: int = 0) -> bool:
        """Bnb4BitLinear::init (Bnb4BitLinear.cpp:453-497) from host checkpoint tensors."""
        return self._create(weight, device, None)

    def init_shard(self, weight: Nf4Tensors, mode: int, rank: int, world: int,
                   device: int = 0) -> bool:
        """Rank ``rank`` of ``world`` of the weight: rows (mode 0) or input columns (mode 1)."""
        return self._create(weight, device, (mode, rank, world))

    def init_from_desc(self, desc: _lib.WeightDesc, shard: tuple[int, int, int] | None = None) -> bool:
        """From a ready descriptor, e.g. ``SafetensorsFile.load_bnb4_weight_ref`` (the
        reference's LoadBnb4BitWeightRef + init pair); ``shard`` = (mode, rank, world). The
        memory the descriptor points to must stay valid until this call returns."""
        return self._create(desc, int(desc.device), shard)

    def _create(self, weight, device, shard) -> bool:
        lib = _lib.load()
        keep: list = []
        d = weight if isinstance(weight, _lib.WeightDesc) else self._desc(weight, device, keep)
        h = ctypes.c_void_p()
        if shard is None:
            st = lib.aila_nf4_linear_create(ctypes.byref(d), ctypes.byref(h))
        else:
            st = lib.aila_nf4_linear_create_shard(ctypes.byref(d), shard[0], shard[1], shard[2],
                                                  ctypes.byref(h))
        if st != _lib.OK:
            self.last_error = lib.aila_nf4_last_error().decode()
            self.last_status = st
            return False
        self.close()
        self._h = h
        self.device = torch.device("cuda", device)
        return True

    def init_fused_rows(self, *sources: "Bnb4BitLinear") -> bool:
        """Bnb4BitLinear::init_fused_rows (Bnb4BitLinear.cpp:499-629): 2..4 sources."""
        lib = _lib.load()
        arr = (ctypes.c_void_p * max(len(sources), 1))(*[s._h for s in sources])
        h = ctypes.c_void_p()
        st = lib.aila_nf4_linear_create_fused_rows(arr, len(sources), ctypes.byref(h))
        if st != _lib.OK:
            self.last_error = lib.aila_nf4_last_error().decode()
            self.last_status = st
            return False
        self.close()
        self._h = h
        self.device = sources[0].device
        return True

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.load().aila_nf4_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- queries ----------------------------------------------------------------------
    def in_features(self) -> int:
        return int(_lib.load().aila_nf4_linear_in_features(self._h))

    def out_features(self) -> int:
        return int(_lib.load().aila_nf4_linear_out_features(self._h))

    def device_bytes(self) -> int:
        return int(_lib.load().aila_nf4_linear_device_bytes(self._h))

    # -- compute ----------------------------------------------------------------------
    def forward(self, scratch: Bnb4BitLinearScratch, input: torch.Tensor, output: torch.Tensor,
                seq_len: int, add_residual: torch.Tensor | None = None) -> None:
        """Bnb4BitLinear::forward (Bnb4BitLinear.cpp:799-949)."""
        if input.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
            raise RuntimeError("Bnb4BitLinear expects bf16 input/output tensors")
        if seq_len <= 0:
            raise RuntimeError("Bnb4BitLinear::forward: seq_len must be positive")
        assert input.is_cuda and output.is_cuda and input.is_contiguous() and output.is_contiguous()
        assert input.numel() >= seq_len * self.in_features()
        assert output.numel() >= seq_len * self.out_features()
        res = add_residual.data_ptr() if add_residual is not None else None
        _lib.check(_lib.load().aila_nf4_forward(self._h, scratch._h, input.data_ptr(),
                                                output.data_ptr(), seq_len, res,
                                                _stream_ptr(self.device)))

    @staticmethod
    def try_forward_decode_gate_up_swiglu(fused_gate_up: "Bnb4BitLinear",
                                          scratch: Bnb4BitLinearScratch, input: torch.Tensor,
                                          output: torch.Tensor, ff_dim: int,
                                          seq_len: int = 1) -> bool:
        """Bnb4BitLinear::try_forward_decode_gate_up_swiglu (Bnb4BitLinear.cpp:759-797); also
        takes seq_len > 1, where it stands for forward + ops::fused_gate_up_swiglu."""
        if input.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
            return False
        if input.dim() != 2:
            return False
        st = _lib.load().aila_nf4_forward_gate_up_swiglu(
            fused_gate_up._h, scratch._h, input.data_ptr(), output.data_ptr(), seq_len, ff_dim,
            _stream_ptr(fused_gate_up.device))
        if st == _lib.NOT_APPLICABLE:
            return False
        _lib.check(st)
        return True

    @staticmethod
    def _norm(weight: torch.Tensor, eps: float, add: torch.Tensor | None,
              hidden_out: torch.Tensor | None) -> _lib.RmsNorm:
        n = _lib.RmsNorm()
        n.add_bf16 = add.data_ptr() if add is not None else None
        n.weight_bf16 = weight.data_ptr()
        n.eps = float(eps)
        n.hidden_out_bf16 = hidden_out.data_ptr() if hidden_out is not None else None
        return n

    def forward_rmsnorm(self, scratch: Bnb4BitLinearScratch, input: torch.Tensor,
                        norm_weight: torch.Tensor, eps: float, output: torch.Tensor,
                        add: torch.Tensor | None = None, hidden_out: torch.Tensor | None = None,
                        add_residual: torch.Tensor | None = None) -> bool:
        """ops::fused_add_rms_norm (NormOps.cpp:141-260) folded into a seq_len == 1 forward:
        the linear sees rmsnorm(input + add) * norm_weight, ``hidden_out`` receives input + add.
        False = not applicable here (run ``add_rms_norm`` and ``forward`` separately)."""
        n = self._norm(norm_weight, eps, add, hidden_out)
        res = add_residual.data_ptr() if add_residual is not None else None
        st = _lib.load().aila_nf4_forward_rmsnorm(self._h, scratch._h, input.data_ptr(),
                                                  ctypes.byref(n), output.data_ptr(), res,
                                                  _stream_ptr(self.device))
        if st == _lib.NOT_APPLICABLE:
            return False
        _lib.check(st)
        return True

    @staticmethod
    def try_forward_decode_gate_up_swiglu_rmsnorm(fused_gate_up: "Bnb4BitLinear",
                                                  scratch: Bnb4BitLinearScratch, input: torch.Tensor,
                                                  norm_weight: torch.Tensor, eps: float,
                                                  output: torch.Tensor, ff_dim: int,
                                                  add: torch.Tensor | None = None,
                                                  hidden_out: torch.Tensor | None = None) -> bool:
        n = Bnb4BitLinear._norm(norm_weight, eps, add, hidden_out)
        st = _lib.load().aila_nf4_forward_gate_up_swiglu_rmsnorm(
            fused_gate_up._h, scratch._h, input.data_ptr(), ctypes.byref(n), output.data_ptr(),
            ff_dim, _stream_ptr(fused_gate_up.device))
        if st == _lib.NOT_APPLICABLE:
            return False
        _lib.check(st)
        return True

    def forward_host(self, scratch: Bnb4BitLinearScratch, x_host: torch.Tensor,
                     y_host: torch.Tensor, seq_len: int) -> None:
        """forward with (pinned) host tensors; copies in, runs, copies out, waits."""
        _lib.check(_lib.load().aila_nf4_forward_host(self._h, scratch._h, x_host.data_ptr(),
                                                     y_host.data_ptr(), seq_len,
                                                     _stream_ptr(self.device)))

    def gate_up_swiglu_host(self, scratch: Bnb4BitLinearScratch, x_host: torch.Tensor,
                            y_host: torch.Tensor, seq_len: int, ff_dim: int) -> None:
        _lib.check(_lib.load().aila_nf4_forward_gate_up_swiglu_host(
            self._h, scratch._h, x_host.data_ptr(), y_host.data_ptr(), seq_len, ff_dim,
            _stream_ptr(self.device)))

    def forward_decode_static(self, input: torch.Tensor, output: torch.Tensor,
                              add_residual: torch.Tensor | None = None) -> None:
        """seq_len == 1 forward on the library's built-in fixed work space: no scratch object
        and no allocation. For hosts that keep the CUDA allocator off their decode loop; calls
        on one GPU must stay on one stream (they share the work space)."""
        if input.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
            raise RuntimeError("Bnb4BitLinear expects bf16 input/output tensors")
        res = add_residual.data_ptr() if add_residual is not None else None
        _lib.check(_lib.load().aila_nf4_forward_decode_static(
            self._h, input.data_ptr(), output.data_ptr(), res, _stream_ptr(self.device)))

    def forward_decode_allreduce(self, scratch: Bnb4BitLinearScratch, peers: "PeerBuffer",
                                 input: torch.Tensor, output: torch.Tensor,
                                 add_residual: torch.Tensor | None = None) -> None:
        """seq_len == 1 forward of a column shard with the sum over ranks folded in: ``input`` is
        this rank's column slice, ``output`` receives the full row sum on every rank."""
        if input.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
            raise RuntimeError("Bnb4BitLinear expects bf16 input/output tensors")
        assert input.is_cuda and output.is_cuda and input.is_contiguous() and output.is_contiguous()
        assert input.numel() >= self.in_features() and output.numel() >= self.out_features()
        res = add_residual.data_ptr() if add_residual is not None else None
        _lib.check(_lib.load().aila_nf4_forward_decode_allreduce(
            self._h, scratch._h, peers._h, input.data_ptr(), output.data_ptr(), res,
            _stream_ptr(self.device)))

    def dequantize_weight(self) -> torch.Tensor:
        """bf16 [in_features, out_features], the transposed layout of
        Bnb4BitLinear::dequantize_weight (Bnb4BitLinear.cpp:723-757)."""
        out = torch.empty(self.in_features(), self.out_features(), dtype=torch.bfloat16,
                          device=self.device)
        _lib.check(_lib.load().aila_nf4_dequantize(self._h, out.data_ptr(), _stream_ptr(self.device)))
        return out

    def dequantize_rowmajor(self) -> torch.Tensor:
        out = torch.empty(self.out_features(), self.in_features(), dtype=torch.bfloat16,
                          device=self.device)
        _lib.check(_lib.load().aila_nf4_dequantize_rowmajor(self._h, out.data_ptr(),
                                                            _stream_ptr(self.device)))
        return out

    def expand_absmax(self, blocksize: int) -> torch.Tensor:
        out = torch.empty(self.out_features(), self.in_features() // blocksize,
                          dtype=torch.float32, device=self.device)
        _lib.check(_lib.load().aila_nf4_expand_absmax(self._h, out.data_ptr(),
                                                      _stream_ptr(self.device)))
        return out


class Linear:
    """Dense bf16 linear (reference class Linear, src/ops/Ops.hpp:16-31): ``init`` with a
    [out_features, in_features] bf16 weight, ``forward(scratch, input, output, seq_len)``."""

    def __init__(self):
        self._h = None
        self.device = None

    def init(self, weight: torch.Tensor, in_features: int, out_features: int, device: int = 0) -> None:
        if weight.dtype != torch.bfloat16 or tuple(weight.shape) != (out_features, in_features):
            raise RuntimeError("Linear::init expects a bf16 [out_features, in_features] weight")
        weight = weight.contiguous()
        h = ctypes.c_void_p()
        _lib.check(_lib.load().aila_dense_linear_create(weight.data_ptr(), out_features, in_features,
                                                        1 if weight.is_cuda else 0, int(device),
                                                        ctypes.byref(h)))
        self.close()
        self._h = h
        self.device = torch.device("cuda", device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.load().aila_dense_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def in_features(self) -> int:
        return int(_lib.load().aila_dense_linear_in_features(self._h))

    def out_features(self) -> int:
        return int(_lib.load().aila_dense_linear_out_features(self._h))

    def forward(self, scratch: Bnb4BitLinearScratch, input: torch.Tensor, output: torch.Tensor,
                seq_len: int, add_residual: torch.Tensor | None = None) -> None:
        if input.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
            raise RuntimeError("Linear expects bf16 input/output tensors")
        assert input.is_cuda and output.is_cuda and input.is_contiguous() and output.is_contiguous()
        assert input.numel() >= seq_len * self.in_features()
        assert output.numel() >= seq_len * self.out_features()
        res = add_residual.data_ptr() if add_residual is not None else None
        _lib.check(_lib.load().aila_dense_linear_forward(self._h, scratch._h, input.data_ptr(),
                                                         output.data_ptr(), seq_len, res,
                                                         _stream_ptr(self.device)))


def add_rms_norm(x: torch.Tensor, add: torch.Tensor | None, weight: torch.Tensor, eps: float,
                 hidden_out: torch.Tensor | None, normed_out: torch.Tensor) -> None:
    """ops::fused_add_rms_norm / rms_norm (NormOps.cpp:141-260) as its own launch, any row count:
    hidden_out = x + add (may alias x), normed_out = rmsnorm(x + add) * weight."""
    rows, hidden = x.shape
    _lib.check(_lib.load().aila_add_rms_norm(
        x.data_ptr(), add.data_ptr() if add is not None else None, weight.data_ptr(), float(eps),
        rows, hidden, hidden_out.data_ptr() if hidden_out is not None else None,
        normed_out.data_ptr(), x.device.index, _stream_ptr(x.device)))


def argmax(logits: torch.Tensor, vocab_size: int, result: torch.Tensor, index_offset: int = 0) -> None:
    """ops::argmax (src/ops/SamplingOps.cpp:321-365): greedy token over bf16 logits, written to
    the int32 device tensor ``result``; equal values resolve as in the reference's reduction (the
    smallest bit-reversed index % 256, then the smallest index). With ``index_offset`` the logits
    are a vocabulary shard starting at that global index: ties are resolved on global indices and
    the result is the local index."""
    assert logits.dtype == torch.bfloat16 and logits.is_cuda and result.dtype == torch.int32
    _lib.check(_lib.load().aila_argmax_bf16_shard(logits.data_ptr(), vocab_size, index_offset, result.data_ptr(),
                                                  logits.device.index, _stream_ptr(logits.device)))


class PeerBuffer:
    """One rank's exchange buffer for ``forward_decode_allreduce`` (aila_nf4_peerbuf_*)."""

    def __init__(self, device: int, rank: int, world: int, max_rows: int):
        self._h = ctypes.c_void_p()
        self.rank, self.world = rank, world
        _lib.check(_lib.load().aila_nf4_peerbuf_create(int(device), rank, world, max_rows,
                                                       ctypes.byref(self._h)))

    def export_handle(self) -> bytes:
        buf = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        _lib.check(_lib.load().aila_nf4_peerbuf_export(self._h, buf))
        return buf.raw

    def import_handle(self, peer_rank: int, handle: bytes) -> None:
        assert len(handle) == _lib.IPC_HANDLE_BYTES
        buf = ctypes.create_string_buffer(handle, _lib.IPC_HANDLE_BYTES)
        _lib.check(_lib.load().aila_nf4_peerbuf_import(self._h, peer_rank, buf))

    def import_local(self, peer_rank: int, peer: "PeerBuffer") -> None:
        """Maps a peer's buffer that this same process created (no IPC handle)."""
        _lib.check(_lib.load().aila_nf4_peerbuf_import_local(self._h, peer_rank, peer._h))
        self._peers = getattr(self, "_peers", []) + [peer]  # keeps the peer's buffer alive

    def close(self) -> None:
        if self._h:
            _lib.load().aila_nf4_peerbuf_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DecodeChain:
    """A run of seq_len == 1 linears executed by ONE launch (aila_nf4_chain_*): the calls the
    reference's decode step makes back to back (Qwen3Bnb4Backend.cpp:400-418). ``ops`` is a list
    of dicts with keys ``linear`` (Bnb4BitLinear), and optionally ``ff_dim`` (> 0: fused gate|up
    + SwiGLU), ``x`` (input tensor; omitted = the previous operation's output), ``y`` (output
    tensor), ``residual`` and ``norm`` = dict(weight=, eps=, add=None, hidden_out=None). With
    ``peers`` (a PeerBuffer whose peers are all imported) the last operation is row-parallel: the
    launch exchanges its row sums with the other ranks and writes the sum (+ residual) to ``y``."""

    def __init__(self, scratch: Bnb4BitLinearScratch, ops: list[dict], peers: "PeerBuffer | None" = None):
        lib = _lib.load()
        self.scratch = scratch
        self.device = scratch.device
        self._keep = []
        arr = (_lib.ChainOp * len(ops))()
        for i, o in enumerate(ops):
            for k in ("x", "y", "residual"):
                tns = o.get(k)
                if tns is not None:
                    assert tns.dtype == torch.bfloat16 and tns.is_cuda and tns.is_contiguous()
                    self._keep.append(tns)
            arr[i].linear = o["linear"]._h
            arr[i].ff_dim = int(o.get("ff_dim", 0))
            arr[i].x_bf16 = o["x"].data_ptr() if o.get("x") is not None else None
            arr[i].y_bf16 = o["y"].data_ptr() if o.get("y") is not None else None
            arr[i].residual_bf16 = o["residual"].data_ptr() if o.get("residual") is not None else None
            nd = o.get("norm")
            if nd is not None:
                n = Bnb4BitLinear._norm(nd["weight"], nd["eps"], nd.get("add"), nd.get("hidden_out"))
                self._keep += [n, nd["weight"], nd.get("add"), nd.get("hidden_out")]
                arr[i].norm = ctypes.pointer(n)
            self._keep.append(o["linear"])
        h = ctypes.c_void_p()
        if peers is None:
            _lib.check(lib.aila_nf4_chain_create(scratch._h, arr, len(ops), ctypes.byref(h)))
        else:  # the last operation is row-parallel: its y is the sum over the ranks
            _lib.check(lib.aila_nf4_chain_create_allreduce(scratch._h, arr, len(ops), peers._h, ctypes.byref(h)))
            self._keep.append(peers)
        self._h = h

    def run(self) -> None:
        _lib.check(_lib.load().aila_nf4_chain_run(self._h, _stream_ptr(self.device)))

    def run_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """x of the first operation from (pinned) host memory, y of the last back to host memory,
        one synchronisation."""
        _lib.check(_lib.load().aila_nf4_chain_run_host(self._h, x_host.data_ptr(), y_host.data_ptr(),
                                                       _stream_ptr(self.device)))

    def __len__(self) -> int:
        return int(_lib.load().aila_nf4_chain_length(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.load().aila_nf4_chain_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def static_check(device: int | torch.device = 0) -> None:
    """Raises if a bounded wait inside a forward_decode_static kernel expired on this GPU since the
    last check (aila_nf4_static_check: reads and clears the status word of the built-in work
    space; allocates nothing)."""
    dev = torch.device("cuda", device) if isinstance(device, int) else device
    _lib.check(_lib.load().aila_nf4_static_check(dev.index or 0, _stream_ptr(dev)))


def set_gemv_kernel(which: int) -> None:
    """0 automatic, 1 plain CUDA-core kernel, 2 streaming kernel with a shared-memory ring,
    3 the chained kernel as a one-operation launch."""
    _lib.check(_lib.load().aila_nf4_set_gemv_kernel(which))
