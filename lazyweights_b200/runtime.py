"""Handles on coded matrices: a whole bundle directory (`Bundle`, the counterpart of the reference runtime's
rt_open handle, kernels/llmrt.cu:1921) or a single blob (`CodedMatrix`).

Host-buffer methods (`matmul`, `decode`, `cpu_decode`) go through the reference-named rt_test_* entry points;
`linear`, `decode_weights` and `decode_codes` take and return CUDA torch tensors and call the device-pointer
entry points on torch's current stream.  torch is only used for device memory and streams.
"""
import ctypes as C
import os

import numpy as np

from . import _native as nat


def _address(a):
    """Address of a contiguous NumPy array's first byte.  `a.ctypes.data_as(...)` costs 4 us, twice per host-buffer call of
    60 us; a ctypes view of the buffer costs 0.6 us (writable arrays only, hence the fallback)."""
    try:
        return C.addressof(C.c_char.from_buffer(a))
    except (TypeError, ValueError, BufferError):
        return a.ctypes.data


def _torch():
    import torch
    return torch


class _Handle:
    def __init__(self, ptr):
        if not ptr:
            raise nat.LwError(nat.lib().lw_last_status() or -1, nat.last_error())
        self._h = C.c_void_p(ptr)
        self._ids = {}
        self._info = {}

    # ---- lifetime
    def close(self):
        if self._h:
            nat.lib().rt_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- lookup
    def matrix_id(self, name):
        if name not in self._ids:
            i = nat.lib().lw_matrix_id(self._h, name.encode())
            if i < 0:
                raise KeyError(name)
            self._ids[name] = i
        return self._ids[name]

    def info(self, name):
        if name in self._info:
            return self._info[name]
        n, k, fmt = C.c_int(), C.c_int(), C.c_int()
        bb, sb, db = C.c_longlong(), C.c_longlong(), C.c_longlong()
        nat.check(nat.lib().lw_matrix_info(self._h, self.matrix_id(name), C.byref(n), C.byref(k), C.byref(fmt),
                                           C.byref(bb), C.byref(sb), C.byref(db)))
        self._info[name] = dict(N=n.value, K=k.value, fmt=nat.FMT_NAME[fmt.value], blob_bytes=bb.value,
                                side_bytes=sb.value, device_bytes=db.value, paired=fmt.value in (1, 4))
        return self._info[name]

    def plan(self, name):
        """How the batch-1 kernel decodes this matrix: {"group", "index_bits", "slow_fraction"}."""
        g, ib, f = C.c_int(), C.c_int(), C.c_double()
        nat.check(nat.lib().lw_matrix_plan(self._h, self.matrix_id(name), C.byref(g), C.byref(ib), C.byref(f)))
        return dict(group=g.value, index_bits=ib.value, slow_fraction=f.value)

    # ---- device-pointer path
    def linear(self, name, x, out=None):
        """x: CUDA tensor [m, K] or [K], fp16 or fp32 -> fp32 [m, N] (or [N])."""
        torch = _torch()
        inf = self.info(name)
        squeeze = x.dim() == 1
        x2 = x.reshape(1, -1) if squeeze else x
        if not x2.is_cuda or x2.dtype not in (torch.float16, torch.float32) or x2.shape[1] != inf["K"]:
            raise ValueError("linear wants a CUDA fp16/fp32 tensor with %d columns" % inf["K"])
        x2 = x2.contiguous()
        m = x2.shape[0]
        y = out if out is not None else torch.empty((m, inf["N"]), dtype=torch.float32, device=x2.device)
        st = torch.cuda.current_stream(x2.device).cuda_stream
        nat.check(nat.lib().lw_linear(self._h, self.matrix_id(name), C.c_void_p(x2.data_ptr()),
                                      int(x2.dtype == torch.float16), m, C.c_void_p(y.data_ptr()), C.c_void_p(st)))
        return y[0] if squeeze and out is None else y

    def linear_static(self, name, x, out):
        """lw_linear_static: the same product with the library's built-in scratch; `out` must be preallocated
        (fp32 [m, N], CUDA) so that the call itself allocates nothing."""
        torch = _torch()
        inf = self.info(name)
        x2 = x.reshape(1, -1) if x.dim() == 1 else x
        if not (x2.is_cuda and x2.is_contiguous() and x2.dtype in (torch.float16, torch.float32)):
            raise ValueError("linear_static wants a contiguous CUDA fp16/fp32 tensor")
        if x2.shape[1] != inf["K"] or tuple(out.shape) != (x2.shape[0], inf["N"]) or out.dtype != torch.float32:
            raise ValueError("shape or dtype mismatch")
        st = torch.cuda.current_stream(x2.device).cuda_stream
        nat.check(nat.lib().lw_linear_static(self._h, self.matrix_id(name), C.c_void_p(x2.data_ptr()),
                                             int(x2.dtype == torch.float16), x2.shape[0], C.c_void_p(out.data_ptr()),
                                             C.c_void_p(st)))
        return out

    # ---- fixed-width twin (the same kernel without Huffman decoding)
    def make_twin(self, name):
        nat.check(nat.lib().lw_matrix_make_twin(self._h, self.matrix_id(name)))
        return True

    def drop_twin(self, name):
        nat.check(nat.lib().lw_matrix_drop_twin(self._h, self.matrix_id(name)))

    def twin_bytes(self, name):
        return int(nat.lib().lw_matrix_twin_bytes(self._h, self.matrix_id(name)))

    def pair_bytes(self, name):
        """Bytes of the matrix's pair layout that a one-row product reads (0: the matrix has none)."""
        return int(nat.lib().lw_matrix_pair_bytes(self._h, self.matrix_id(name)))

    def linear_twin(self, name, x, out=None):
        """y[N] = W x for one activation row, read from the twin (make_twin first)."""
        torch = _torch()
        inf = self.info(name)
        x2 = x.reshape(1, -1).contiguous()
        if not x2.is_cuda or x2.dtype not in (torch.float16, torch.float32) or x2.shape[1] != inf["K"]:
            raise ValueError("linear_twin wants one CUDA fp16/fp32 row with %d columns" % inf["K"])
        y = out if out is not None else torch.empty((1, inf["N"]), dtype=torch.float32, device=x2.device)
        st = torch.cuda.current_stream(x2.device).cuda_stream
        nat.check(nat.lib().lw_linear_twin(self._h, self.matrix_id(name), C.c_void_p(x2.data_ptr()),
                                           int(x2.dtype == torch.float16), C.c_void_p(y.data_ptr()), C.c_void_p(st)))
        return y

    def decode_weights(self, name, out=None):
        """fp16 CUDA tensor [N, K] of the dequantised weights (`out`: a contiguous tensor of that shape to fill)."""
        torch = _torch()
        inf = self.info(name)
        w = out if out is not None else torch.empty((inf["N"], inf["K"]), dtype=torch.float16, device="cuda")
        if w.dtype != torch.float16 or tuple(w.shape) != (inf["N"], inf["K"]) or not w.is_cuda or not w.is_contiguous():
            raise ValueError("decode_weights wants a contiguous CUDA fp16 [%d, %d] tensor" % (inf["N"], inf["K"]))
        st = torch.cuda.current_stream().cuda_stream
        nat.check(nat.lib().lw_decode_weights(self._h, self.matrix_id(name), C.c_void_p(w.data_ptr()), C.c_void_p(st)))
        return w

    def decode_codes(self, name, expand=True, out=None):
        """uint8 CUDA tensor: codes [N, K] (expand) or symbols [N, K / 2] of a paired matrix (`out`: a contiguous tensor
        of that shape to fill)."""
        torch = _torch()
        inf = self.info(name)
        cols = inf["K"] if (expand or not inf["paired"]) else inf["K"] // 2
        if out is None:
            out = torch.empty((inf["N"], cols), dtype=torch.uint8, device="cuda")
        if out.dtype != torch.uint8 or tuple(out.shape) != (inf["N"], cols) or not out.is_cuda or not out.is_contiguous():
            raise ValueError("decode_codes wants a contiguous CUDA uint8 [%d, %d] tensor" % (inf["N"], cols))
        st = torch.cuda.current_stream().cuda_stream
        nat.check(nat.lib().lw_decode_codes(self._h, self.matrix_id(name), C.c_void_p(out.data_ptr()), int(expand),
                                            C.c_void_p(st)))
        return out

    # ---- host-buffer path (reference-named entry points)
    def matmul(self, name, X, path=0):
        """Y[m, N] = X[m, K] . W^T with host float32 arrays (rt_test_matmul)."""
        X = np.ascontiguousarray(np.atleast_2d(X), np.float32)
        inf = self.info(name)
        if X.shape[1] != inf["K"]:
            raise ValueError("X has %d columns, the matrix %d" % (X.shape[1], inf["K"]))
        Y = np.empty((X.shape[0], inf["N"]), np.float32)
        nat.check(nat.lib().rt_test_matmul(self._h, name.encode(), _address(X), X.shape[0], _address(Y), path))
        return Y

    def decode(self, name):
        """uint8 [N, K] codes on the host (rt_test_decode)."""
        inf = self.info(name)
        out = np.empty((inf["N"], inf["K"]), np.uint8)
        nat.check(nat.lib().rt_test_decode(self._h, name.encode(), out.ctypes.data_as(C.c_void_p)))
        return out

    def kernel_error(self):
        return nat.lib().lw_kernel_error()


class ProductBatch:
    """A fixed list of one-row products y_j = W_j x_j prepared once and launched together (lw_linear_batch): up to
    eight products per kernel launch where the matrices share format and decode plan.  entries: (handle, matrix
    name, x CUDA tensor [K], y CUDA fp32 tensor [N]); all x of one dtype (fp16 or fp32).  The tensors are kept alive."""

    def __init__(self, entries):
        torch = _torch()
        self._keep = list(entries)
        n = len(self._keep)
        if n == 0:
            raise ValueError("empty batch")
        half = self._keep[0][2].dtype == torch.float16
        self._n, self._half = n, int(half)
        self._handles = (C.c_void_p * n)()
        self._ids = (C.c_int * n)()
        self._xs = (C.c_void_p * n)()
        self._ys = (C.c_void_p * n)()
        for j, (h, name, x, y) in enumerate(self._keep):
            inf = h.info(name)
            if not (x.is_cuda and y.is_cuda and x.is_contiguous() and y.is_contiguous() and y.dtype == torch.float32 and
                    x.numel() == inf["K"] and y.numel() == inf["N"] and (x.dtype == torch.float16) == half and
                    x.dtype in (torch.float16, torch.float32)):
                raise ValueError("entry %d: wrong shape, dtype or device" % j)
            self._handles[j], self._ids[j] = h._h.value, h.matrix_id(name)
            self._xs[j], self._ys[j] = x.data_ptr(), y.data_ptr()

    def launch(self):
        st = _torch().cuda.current_stream().cuda_stream
        nat.check(nat.lib().lw_linear_batch(self._n, self._handles, self._ids, self._xs, self._half, self._ys, C.c_void_p(st)))


class Bundle(_Handle):
    """A bundle directory opened on the current CUDA device."""

    def __init__(self, path, max_ctx=4096, max_batch=8, verbose=False):
        self.path = path
        super().__init__(nat.lib().rt_open(os.fsencode(path), max_ctx, max_batch, -1, 0, int(verbose)))

    # ---- decoder runtime (bundles with a model cfg)
    def forward(self, ids, all_logits=False):
        """rt_forward: logits of the last token [vocab] or of every token [n, vocab] (host float32)."""
        ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
        v = nat.lib().rt_vocab(self._h)
        out = np.empty((ids.size, v) if all_logits else (v,), np.float32)
        rc = nat.lib().rt_forward(self._h, ids.ctypes.data_as(C.c_void_p), ids.size, out.ctypes.data_as(C.c_void_p),
                                  int(all_logits))
        if rc == -1:
            raise IndexError("context overflow")
        nat.check(rc)
        return out

    def decode_greedy(self, first_token, n):
        """rt_decode_greedy: n greedy one-token passes without a host round trip per token; returns the n chosen tokens
        (int32).  The same tokens as n calls of forward() with np.argmax in between."""
        out = np.empty(n, np.int32)
        rc = nat.lib().rt_decode_greedy(self._h, int(first_token), int(n), out.ctypes.data_as(C.c_void_p))
        if rc == -1:
            raise IndexError("context overflow")
        nat.check(rc)
        return out

    def reset(self):
        nat.lib().rt_reset(self._h)

    def set_pos(self, p):
        nat.lib().rt_set_pos(self._h, p)

    def set_window(self, w):
        nat.lib().rt_set_window(self._h, w)

    @property
    def pos(self):
        return nat.lib().rt_pos(self._h)

    @property
    def vocab(self):
        return nat.lib().rt_vocab(self._h)

    def tp_init(self, rank, world, unique_id):
        nat.check(nat.lib().rt_tp_init(self._h, rank, world, (C.c_uint8 * 128).from_buffer_copy(unique_id)))

    def tp_peer_export(self):
        buf = (C.c_uint8 * 64)()
        nat.check(nat.lib().rt_tp_peer_export(self._h, buf))
        return bytes(buf)

    def tp_peer_open(self, handles, world):
        nat.check(nat.lib().rt_tp_peer_open(self._h, (C.c_uint8 * (64 * world)).from_buffer_copy(handles), world))

    def tp_error(self):
        return nat.lib().rt_tp_error(self._h)

    def tp_set_timeout(self, timeout_ms):
        """Bound (ms) on the wait for a tensor-parallel pass: after it the communicator is aborted and the call fails
        (0: LW_TP_TIMEOUT_MS or 60 s)."""
        nat.check(nat.lib().rt_tp_set_timeout(self._h, int(timeout_ms)))

    def debug_stream_stall(self, ms):
        """Test hook: the stream is held up for `ms` milliseconds by a sleeping host function, then the bounded wait
        runs; returns 0 if it saw the stream drain, a negative status if it gave up first."""
        return nat.lib().lw_debug_stream_stall(self._h, int(ms))

    def cpu_decode(self, name, threads=0):
        inf = self.info(name)
        cols = inf["K"] // 2 if inf["paired"] else inf["K"]
        out = np.empty((inf["N"], cols), np.uint8)
        nat.check(nat.lib().rt_test_cpu_decode(self._h, name.encode(), threads or (os.cpu_count() or 1),
                                               out.ctypes.data_as(C.c_void_p)))
        return out

    def stat(self, key):
        return nat.lib().rt_stat(self._h, key.encode())

    def gpu_decode_all(self, reps=3):
        return nat.lib().rt_gpu_decode_all(self._h, reps)

    def cpu_decode_all(self, threads=0):
        n = C.c_longlong(0)
        s = nat.lib().rt_cpu_decode_all(self._h, threads or (os.cpu_count() or 1), C.byref(n))
        return s, n.value


def tp_unique_id():
    buf = (C.c_uint8 * 128)()
    nat.check(nat.lib().lw_tp_unique_id(buf))
    return bytes(buf)


class CodedMatrix(_Handle):
    """One blob (N rows, Ks symbols per row) with an optional side tensor of block format `fmt`."""
    NAME = "m"

    def __init__(self, blob, N, Ks, fmt="none", side=None):
        b = np.frombuffer(blob, np.uint8)
        s = np.ascontiguousarray(side, np.uint8).reshape(-1) if side is not None else np.zeros(0, np.uint8)
        super().__init__(nat.lib().lw_matrix_create(b.ctypes.data_as(C.c_void_p), b.size, N, Ks, nat.FMT[fmt],
                                                    s.ctypes.data_as(C.c_void_p) if s.size else None, s.size))

    def decode_symbols(self):
        return self.decode_codes(self.NAME, expand=False).cpu().numpy()
