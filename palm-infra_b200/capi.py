"""ctypes binding of libb200w4.so, the C-ABI library declared in include/b200w4.h.

This is the only route from Python to the kernels.  There is no CPU fallback: importing
works anywhere (so the library's exports can be checked without a GPU), but creating a
Context raises unless an sm_100 device and the built library are present.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200w4.so")

ACT_G128, ACT_G32 = 128, 32
NONE, SILU, GELU, RELU, RELU_SQUARED = 0, 1, 2, 3, 4

# every symbol include/b200w4.h declares
SYMBOLS = [
    "b2w4_ctx_create", "b2w4_ctx_destroy", "b2w4_ctx_set_stream", "b2w4_sync",
    "b2w4_ctx_set_peer_wait_ms", "b2w4_ctx_set_moe_rule",
    "b2w4_last_error", "b2w4_version", "b2w4_weight_upload", "b2w4_weight_from_device",
    "b2w4_weight_free", "b2w4_weight_shape", "b2w4_weight_scales_fp16",
    "b2w4_weight_stream_bytes", "b2w4_matmul", "b2w4_matmul_host",
    "b2w4_matmul_static_scratch",
    "b2w4_debug_group_sums", "b2w4_quantize_activations", "b2w4_moe_forward",
    "b2w4_moe_select_routes", "b2w4_moe_expert_outputs", "b2w4_moe_combine",
    "b2w4_matmul_tp", "b2w4_tp_gather", "b2w4_moe_forward_ep", "b2w4_matmul_argmax",
    "b2w4_matmul_argmax_tp", "b2w4_tp_gather_token",
    "b2w4_chain_create", "b2w4_chain_create_tp", "b2w4_chain_scratch_words", "b2w4_chain_destroy", "b2w4_chain_run", "b2w4_chain_run_host",
    "b2w4_chain_input", "b2w4_chain_output", "b2w4_chain_weight_bytes", "b2w4_chain_set_trace",
    "b2w4_rms_norm", "b2w4_add_rms_norm", "b2w4_swiglu", "b2w4_elementwise", "b2w4_rope",
    "b2w4_attention", "b2w4_embed_rows", "b2w4_copy_rows", "b2w4_advance",
    "b2w4_qkv_prepare", "b2w4_rope_tables",
    "b2w4_kernel_launches",
]

_lib = None


class TpGroup(C.Structure):
    """b2w4_tp_group: this rank, the world size, and every rank's staging buffer
    (uint64[2 + 2 * half], zeroed, 16-byte aligned; half = 8 * ldc for matmul_tp) as mapped into this process (peer pointers)."""
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("stage_peers", C.c_void_p * 8)]


class ChainOp(C.Structure):
    """b2w4_chain_op: one GEMV of a list run as one persistent kernel."""
    _fields_ = [("w", C.c_void_p), ("x_from", C.c_int), ("x_offset", C.c_int),
                ("x_dev", C.c_void_p), ("y_dev", C.c_void_p), ("activation", C.c_int),
                ("act_n_begin", C.c_int), ("act_n_len", C.c_int)]


class ChainShard(C.Structure):
    """b2w4_chain_shard: which columns of the full row this rank's shard of an op holds, and
    (optionally) every rank's plain fp32 row as mapped into this process."""
    _fields_ = [("n_offset", C.c_int), ("n_full", C.c_int), ("y_peers", C.c_void_p * 8)]


class B200W4Error(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200W4Error(
                f"{LIB_PATH} is missing: build it with `python palm-infra_b200/build.py`; "
                "there is no fallback path")
        L = C.CDLL(LIB_PATH)
        vp, i, f_p = C.c_void_p, C.c_int, C.c_void_p
        L.b2w4_ctx_create.argtypes = [i, C.POINTER(vp)]
        L.b2w4_ctx_destroy.argtypes = [vp]
        L.b2w4_ctx_destroy.restype = None
        L.b2w4_ctx_set_stream.argtypes = [vp, vp]
        L.b2w4_sync.argtypes = [vp]
        L.b2w4_ctx_set_peer_wait_ms.argtypes = [vp, i]
        L.b2w4_ctx_set_moe_rule.argtypes = [vp, i]
        L.b2w4_last_error.argtypes = [vp]
        L.b2w4_last_error.restype = C.c_char_p
        L.b2w4_version.restype = C.c_char_p
        L.b2w4_weight_upload.argtypes = [vp, vp, i, i, C.POINTER(vp)]
        L.b2w4_weight_from_device.argtypes = [vp, vp, i, i, C.POINTER(vp)]
        L.b2w4_weight_free.argtypes = [vp, vp]
        L.b2w4_weight_free.restype = None
        L.b2w4_weight_shape.argtypes = [vp, C.POINTER(i), C.POINTER(i)]
        L.b2w4_weight_scales_fp16.argtypes = [vp]
        L.b2w4_weight_stream_bytes.argtypes = [vp]
        L.b2w4_weight_stream_bytes.restype = C.c_size_t
        L.b2w4_matmul.argtypes = [vp, vp, f_p, i, f_p, i, i, i, i, i, i]
        L.b2w4_matmul_host.argtypes = [vp, vp, f_p, i, f_p, i, i, i, i, i, i]
        L.b2w4_matmul_static_scratch.argtypes = [vp, vp, f_p, i, f_p, i, i, i, i, i]
        L.b2w4_debug_group_sums.argtypes = [vp, vp, f_p, i, i, i, vp]
        L.b2w4_quantize_activations.argtypes = [vp, f_p, i, i, i, i, vp, vp]
        L.b2w4_moe_forward.argtypes = [vp, f_p, i, i, i, vp, i, i, i, vp, vp, f_p, i, f_p,
                                       vp, f_p]
        L.b2w4_moe_select_routes.argtypes = [vp, f_p, i, i, i, vp, f_p]
        L.b2w4_moe_expert_outputs.argtypes = [vp, f_p, i, i, i, vp, i, i, i, vp, vp, i, i, f_p,
                                              vp, f_p]
        L.b2w4_moe_combine.argtypes = [vp, f_p, i, i, i, vp, f_p, f_p, i]
        L.b2w4_matmul_tp.argtypes = [vp, vp, f_p, i, i, i, i, C.POINTER(TpGroup), i, i, i]
        L.b2w4_tp_gather.argtypes = [vp, C.POINTER(TpGroup), f_p, i, i]
        L.b2w4_matmul_argmax.argtypes = [vp, vp, f_p, i, i, f_p, i, vp]
        L.b2w4_matmul_argmax_tp.argtypes = [vp, vp, f_p, i, i, i, C.POINTER(TpGroup)]
        L.b2w4_tp_gather_token.argtypes = [vp, C.POINTER(TpGroup), vp, i]
        L.b2w4_moe_forward_ep.argtypes = [vp, f_p, i, i, i, vp, i, i, i, vp, vp, i, i,
                                          C.POINTER(TpGroup), i, f_p, i, vp, f_p]
        L.b2w4_chain_create.argtypes = [vp, C.POINTER(ChainOp), i, C.POINTER(vp)]
        L.b2w4_chain_create_tp.argtypes = [vp, C.POINTER(ChainOp), C.POINTER(ChainShard), i,
                                           C.POINTER(TpGroup), C.POINTER(vp)]
        L.b2w4_chain_scratch_words.argtypes = [C.POINTER(ChainShard), i]
        L.b2w4_chain_scratch_words.restype = C.c_size_t
        L.b2w4_chain_destroy.argtypes = [vp, vp]
        L.b2w4_chain_destroy.restype = None
        L.b2w4_chain_run.argtypes = [vp, vp]
        L.b2w4_chain_run_host.argtypes = [vp, vp, f_p, i, f_p, i]
        L.b2w4_chain_set_trace.argtypes = [vp, vp, i]
        L.b2w4_chain_input.argtypes = [vp]
        L.b2w4_chain_input.restype = C.c_void_p
        L.b2w4_chain_output.argtypes = [vp]
        L.b2w4_chain_output.restype = C.c_void_p
        L.b2w4_chain_weight_bytes.argtypes = [vp]
        L.b2w4_chain_weight_bytes.restype = C.c_size_t
        fl = C.c_float
        L.b2w4_rms_norm.argtypes = [vp, f_p, i, i, i, f_p, fl, f_p, i]
        L.b2w4_add_rms_norm.argtypes = [vp, f_p, i, f_p, i, i, i, f_p, fl, f_p, i]
        L.b2w4_swiglu.argtypes = [vp, f_p, i, i, i, f_p, i]
        L.b2w4_elementwise.argtypes = [vp, f_p, f_p, f_p, C.c_size_t, i]
        L.b2w4_rope.argtypes = [vp, f_p, f_p, i, i, i, f_p, f_p, i, i, vp]
        L.b2w4_attention.argtypes = [vp, f_p, f_p, f_p, f_p, f_p, f_p, i, i, i, i, i, vp, i, fl]
        L.b2w4_advance.argtypes = [vp, vp, i, vp, vp, i]
        L.b2w4_rope_tables.argtypes = [vp, vp, i, i, i, fl]
        L.b2w4_qkv_prepare.argtypes = [vp, f_p, i, i, i, i, i, f_p, f_p, fl, f_p, f_p, i, vp,
                                       f_p, f_p, f_p, i]
        L.b2w4_embed_rows.argtypes = [vp, vp, vp, i, i, f_p, i]
        L.b2w4_copy_rows.argtypes = [vp, f_p, i, f_p, i, i, i]
        L.b2w4_kernel_launches.argtypes = [vp]
        L.b2w4_kernel_launches.restype = C.c_uint64
        _lib = L
    return _lib


def _dptr(t):
    """Device pointer of a torch CUDA tensor (or None)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def rope_tables(positions, first_position, rope_dim, theta):
    """(cos, sin) [positions, rope_dim // 2] on the host, as the reference's engine fills them
    (b2w4_rope_tables); needs no GPU."""
    import numpy as np
    cos = np.zeros((positions, rope_dim // 2), dtype=np.float32)
    sin = np.zeros_like(cos)
    rc = lib().b2w4_rope_tables(cos.ctypes.data, sin.ctypes.data, positions, first_position,
                                rope_dim, theta)
    if rc != 0:
        raise B200W4Error(f"b2w4_rope_tables: error {rc}")
    return cos, sin


class Weight:
    def __init__(self, ctx, handle, n, k):
        self.ctx, self.handle, self.n, self.k = ctx, handle, n, k

    @property
    def scales_fp16(self):
        return bool(lib().b2w4_weight_scales_fp16(self.handle))

    @property
    def stream_bytes(self):
        return int(lib().b2w4_weight_stream_bytes(self.handle))

    def free(self):
        if self.handle:
            lib().b2w4_weight_free(self.ctx.handle, self.handle)
            self.handle = None


class Chain:
    """A list of one-row GEMVs compiled into one persistent kernel (b2w4_chain_*).
    ops: list of dicts with keys w (Weight), and optionally x_from, x_offset, x (torch
    tensor), y (torch tensor), act, act_begin, act_len."""

    @staticmethod
    def shard_table(shards):
        """shards: list of (n_offset, n_full, [y_peer pointers or None]) -> ChainShard array."""
        arr = (ChainShard * len(shards))()
        for i, (off, full, peers) in enumerate(shards):
            arr[i].n_offset, arr[i].n_full = off, full
            for p, ptr in enumerate(peers or []):
                arr[i].y_peers[p] = ptr
        return arr

    @staticmethod
    def scratch_words(shard_arr):
        return int(lib().b2w4_chain_scratch_words(shard_arr, len(shard_arr)))

    def __init__(self, ctx, ops, shards=None, group=None):
        """shards (a ChainShard array from shard_table) and group (TpGroup whose stage_peers are
        every rank's zeroed scratch of scratch_words(shards) uint64) select the tensor-parallel
        form."""
        self.ctx = ctx
        arr = (ChainOp * len(ops))()
        self.keep = [shards, group]
        for i, o in enumerate(ops):
            arr[i].w = o["w"].handle
            arr[i].x_from = o.get("x_from", -1)
            arr[i].x_offset = o.get("x_offset", 0)
            x, y = o.get("x"), o.get("y")
            arr[i].x_dev = x.data_ptr() if x is not None else None
            arr[i].y_dev = y.data_ptr() if y is not None else None
            arr[i].activation = o.get("act", NONE)
            arr[i].act_n_begin = o.get("act_begin", 0)
            arr[i].act_n_len = o.get("act_len", -1)
            self.keep.append((o["w"], x, y))
        h = C.c_void_p()
        if group is None:
            ctx._check(lib().b2w4_chain_create(ctx.handle, arr, len(ops), C.byref(h)))
        else:
            ctx._check(lib().b2w4_chain_create_tp(ctx.handle, arr, shards, len(ops),
                                                  C.byref(group), C.byref(h)))
        self.handle = h
        self.count = len(ops)

    def run(self):
        self.ctx._check(lib().b2w4_chain_run(self.ctx.handle, self.handle))

    def run_host(self, x_np, y_np):
        self.ctx._check(lib().b2w4_chain_run_host(
            self.ctx.handle, self.handle,
            x_np.ctypes.data_as(C.c_void_p) if x_np is not None else None,
            x_np.size if x_np is not None else 0,
            y_np.ctypes.data_as(C.c_void_p) if y_np is not None else None,
            y_np.size if y_np is not None else 0))

    def bind_run_host(self, x_np, y_np):
        """run_host with its arguments resolved once (for timing loops)."""
        fn, ch, h = lib().b2w4_chain_run_host, self.handle, self.ctx.handle
        args = (h, ch, x_np.ctypes.data, x_np.size, y_np.ctypes.data, y_np.size)
        keep = (x_np, y_np)

        def call():
            rc = fn(*args)
            if rc != 0:
                self.ctx._check(rc)
            return keep
        return call

    def set_trace(self, trace, cta=0):
        """trace: int64 CUDA tensor [ops, 8] (or None to switch the profiling hook off)."""
        self.ctx._check(lib().b2w4_chain_set_trace(self.handle, _dptr(trace), cta))
        self.keep.append(trace)

    @property
    def input_ptr(self):
        return lib().b2w4_chain_input(self.handle)

    @property
    def output_ptr(self):
        return lib().b2w4_chain_output(self.handle)

    @property
    def weight_bytes(self):
        return int(lib().b2w4_chain_weight_bytes(self.handle))

    def free(self):
        if self.handle:
            lib().b2w4_chain_destroy(self.ctx.handle, self.handle)
            self.handle = None


class Context:
    """One per GPU.  Mirrors what the reference's CudaBackend keeps per device."""

    def __init__(self, device=0):
        h = C.c_void_p()
        rc = lib().b2w4_ctx_create(device, C.byref(h))
        if rc != 0:
            raise B200W4Error(f"b2w4_ctx_create(device={device}) failed with {rc}: "
                              "an sm_100 (B200) device is required; there is no CPU path")
        self.handle = h
        self.device = device

    def _check(self, rc):
        if rc != 0:
            raise B200W4Error(f"b200w4 error {rc}: "
                              f"{lib().b2w4_last_error(self.handle).decode()}")

    def close(self):
        if self.handle:
            lib().b2w4_ctx_destroy(self.handle)
            self.handle = None

    def set_stream(self, cuda_stream_ptr):
        self._check(lib().b2w4_ctx_set_stream(self.handle, C.c_void_p(cuda_stream_ptr)))

    def sync(self):
        self._check(lib().b2w4_sync(self.handle))

    def set_moe_rule(self, rule):
        """ACT_G32: the reference's rule (per 32 values for an expert that holds several rows,
        per 128 for a lone row); ACT_G128: per 128 for every row."""
        self._check(lib().b2w4_ctx_set_moe_rule(self.handle, rule))

    def set_peer_wait_ms(self, milliseconds):
        """Bound of the device-side waits for another GPU's stores (default about 2 s)."""
        self._check(lib().b2w4_ctx_set_peer_wait_ms(self.handle, int(milliseconds)))

    @property
    def launches(self):
        return int(lib().b2w4_kernel_launches(self.handle))

    # -- weights
    def upload_weight(self, host_blocks, n, k):
        """host_blocks: numpy uint8 array of canonical BG128 blocks."""
        h = C.c_void_p()
        self._check(lib().b2w4_weight_upload(self.handle,
                                             host_blocks.ctypes.data_as(C.c_void_p), n, k,
                                             C.byref(h)))
        return Weight(self, h, n, k)

    def weight_from_device(self, dev_blocks, n, k):
        h = C.c_void_p()
        self._check(lib().b2w4_weight_from_device(self.handle, _dptr(dev_blocks), n, k,
                                                  C.byref(h)))
        return Weight(self, h, n, k)

    # -- matmul on device tensors (torch, fp32, row-major [M,K] / [M,N])
    def matmul(self, w, x, y, m=None, rule=ACT_G128, act=NONE, act_begin=0, act_len=-1,
               lda=None, ldc=None):
        m = x.shape[0] if m is None else m
        lda = x.stride(0) if lda is None else lda
        ldc = y.stride(0) if ldc is None else ldc
        self._check(lib().b2w4_matmul(self.handle, w.handle, _dptr(x), lda, _dptr(y), ldc,
                                      m, rule, act, act_begin, act_len))

    def matmul_static_scratch(self, w, x, y, m=None, act=NONE, act_begin=0, act_len=-1):
        """The tensor-core matmul with its scratch in the library's fixed device array
        (5 <= M <= 256, K <= 10240): allocates nothing.  The first call on a device does a
        one-time address look-up, so make it before any stream capture; overlapping calls
        race on the shared array."""
        m = x.shape[0] if m is None else m
        self._check(lib().b2w4_matmul_static_scratch(self.handle, w.handle, _dptr(x),
                                                     x.stride(0), _dptr(y), y.stride(0), m,
                                                     act, act_begin, act_len))

    def matmul_host(self, w, x_np, y_np, rule=ACT_G128, act=NONE, act_begin=0, act_len=-1):
        m = x_np.shape[0]
        self._check(lib().b2w4_matmul_host(
            self.handle, w.handle, x_np.ctypes.data_as(C.c_void_p), x_np.strides[0] // 4,
            y_np.ctypes.data_as(C.c_void_p), y_np.strides[0] // 4, m, rule, act, act_begin,
            act_len))

    def bind_matmul_host(self, w, x_np, y_np, rule=ACT_G128, act=NONE, act_begin=0, act_len=-1):
        """The same call with its arguments resolved once: returns a function of no arguments
        for loops that repeat it (pointer extraction from numpy costs as much as the call)."""
        fn = lib().b2w4_matmul_host
        args = (self.handle, w.handle, x_np.ctypes.data, x_np.strides[0] // 4,
                y_np.ctypes.data, y_np.strides[0] // 4, x_np.shape[0], rule, act, act_begin,
                act_len)
        keep = (w, x_np, y_np)

        def call():
            rc = fn(*args)
            if rc != 0:
                self._check(rc)
            return keep[2]
        return call

    def matmul_tp(self, w_shard, x, ldc, n_offset, group, act=NONE, act_begin=0, act_len=-1):
        """Matmul of up to 8 rows x [m, K] whose epilogue stores this rank's output columns
        into every rank's staging buffer."""
        self._check(lib().b2w4_matmul_tp(self.handle, w_shard.handle, _dptr(x), x.stride(0),
                                         x.shape[0], ldc, n_offset, C.byref(group), act,
                                         act_begin, act_len))

    def matmul_argmax(self, w, x, tokens, y=None):
        """Matmul of up to 8 rows whose epilogue picks each row's greedy token (int32 tokens
        [m] on the device); the logits are written only when y is given."""
        self._check(lib().b2w4_matmul_argmax(
            self.handle, w.handle, _dptr(x), x.stride(0), x.shape[0],
            _dptr(y) if y is not None else None, y.stride(0) if y is not None else 0,
            _dptr(tokens)))

    def matmul_argmax_tp(self, w_shard, x, n_offset, group):
        """This rank's half of the tensor-parallel greedy token (see tp_gather_token)."""
        self._check(lib().b2w4_matmul_argmax_tp(self.handle, w_shard.handle, _dptr(x),
                                                x.stride(0), x.shape[0], n_offset,
                                                C.byref(group)))

    def tp_gather_token(self, group, tokens):
        self._check(lib().b2w4_tp_gather_token(self.handle, C.byref(group), _dptr(tokens),
                                               tokens.shape[0]))

    def tp_gather(self, group, y, ldc):
        """Wait for every rank's values of the latest matmul_tp and unpack them into y."""
        self._check(lib().b2w4_tp_gather(self.handle, C.byref(group), _dptr(y), y.shape[0],
                                         ldc))

    def group_sums(self, w, x, sums, rule=ACT_G128):
        self._check(lib().b2w4_debug_group_sums(self.handle, w.handle, _dptr(x),
                                                x.stride(0), x.shape[0], rule, _dptr(sums)))

    def quantize(self, x, q, scales, rule=ACT_G128):
        self._check(lib().b2w4_quantize_activations(self.handle, _dptr(x), x.stride(0),
                                                    x.shape[0], x.shape[1], rule, _dptr(q),
                                                    _dptr(scales)))

    # -- the operators between a decoder layer's matmuls (torch CUDA tensors, fp32)
    def rms_norm(self, x, weight, eps, out):
        rows, dim = x.shape
        self._check(lib().b2w4_rms_norm(self.handle, _dptr(x), x.stride(0), rows, dim,
                                        _dptr(weight), eps, _dptr(out), out.stride(0)))

    def add_rms_norm(self, residual, update, weight, eps, out):
        rows, dim = residual.shape
        self._check(lib().b2w4_add_rms_norm(self.handle, _dptr(residual), residual.stride(0),
                                            _dptr(update), update.stride(0), rows, dim,
                                            _dptr(weight), eps, _dptr(out), out.stride(0)))

    def swiglu(self, merged, out):
        rows, two_i = merged.shape
        self._check(lib().b2w4_swiglu(self.handle, _dptr(merged), merged.stride(0), rows,
                                      two_i // 2, _dptr(out), out.stride(0)))

    def add(self, a, b, out, multiply=False):
        self._check(lib().b2w4_elementwise(self.handle, _dptr(a), _dptr(b), _dptr(out),
                                           a.numel(), 1 if multiply else 0))

    def rope(self, x, out, tokens, heads, dim, cos, sin, rope_dim, first_position=0,
             position_dev=None):
        """cos / sin: tables [positions, rope_dim // 2]; token t takes row first_position + t,
        or position_dev[0] + t (an int32 CUDA tensor)."""
        self._check(lib().b2w4_rope(self.handle, _dptr(x), _dptr(out), tokens, heads, dim,
                                    _dptr(cos), _dptr(sin), rope_dim, first_position,
                                    _dptr(position_dev)))

    def attention(self, q, k, v, k_cache, v_cache, out, tokens, heads, kv_heads, dim, past,
                  capacity, scale, past_dev=None):
        self._check(lib().b2w4_attention(self.handle, _dptr(q), _dptr(k), _dptr(v),
                                         _dptr(k_cache), _dptr(v_cache), _dptr(out), tokens,
                                         heads, kv_heads, dim, past, _dptr(past_dev), capacity,
                                         scale))

    def qkv_prepare(self, qkv, tokens, heads, kv_heads, dim, q_weight, k_weight, eps, cos, sin,
                    past, q_out, k_cache, v_cache, capacity, past_dev=None):
        """Merged qkv rows -> normalised + rotated Q in q_out, K and V in their cache rows."""
        self._check(lib().b2w4_qkv_prepare(
            self.handle, _dptr(qkv), qkv.stride(0), tokens, heads, kv_heads, dim,
            _dptr(q_weight), _dptr(k_weight), eps, _dptr(cos), _dptr(sin), past, _dptr(past_dev),
            _dptr(q_out), _dptr(k_cache), _dptr(v_cache), capacity))

    def advance(self, counter_dev, by=1, token_dev=None, history_dev=None):
        """counter_dev[0] += by after history_dev[counter_dev[0]] = token_dev[0]."""
        self._check(lib().b2w4_advance(self.handle, _dptr(counter_dev), by, _dptr(token_dev),
                                       _dptr(history_dev),
                                       history_dev.numel() if history_dev is not None else 0))

    def copy_rows(self, src, dst, rows, cols):
        """dst[r, :cols] = src[r, :cols]; src / dst are 2-D views with their own row strides."""
        self._check(lib().b2w4_copy_rows(self.handle, _dptr(src), src.stride(0), _dptr(dst),
                                         dst.stride(0), rows, cols))

    def embed_rows(self, table_fp16, ids, out):
        rows, dim = out.shape
        self._check(lib().b2w4_embed_rows(self.handle, _dptr(table_fp16), _dptr(ids), rows, dim,
                                          _dptr(out), out.stride(0)))

    # -- MoE
    def moe_forward(self, hidden, router_fp16, top_k, intermediate, gate_up, down, out,
                    logits=None, indices=None, weights=None):
        t, h = hidden.shape
        e = router_fp16.shape[0]
        self._check(lib().b2w4_moe_forward(
            self.handle, _dptr(hidden), hidden.stride(0), t, h, _dptr(router_fp16), e, top_k,
            intermediate, gate_up.handle, down.handle, _dptr(out), out.stride(0),
            _dptr(logits), _dptr(indices), _dptr(weights)))

    def moe_expert_outputs(self, hidden, router_fp16, top_k, intermediate, gate_up_local,
                           down_local, expert_begin, expert_count, route_out, indices, weights):
        """One rank's half of the expert-parallel MoE op: route_out [tokens*top_k, H]."""
        t, h = hidden.shape
        e = router_fp16.shape[0]
        self._check(lib().b2w4_moe_expert_outputs(
            self.handle, _dptr(hidden), hidden.stride(0), t, h, _dptr(router_fp16), e, top_k,
            intermediate, gate_up_local.handle, down_local.handle, expert_begin, expert_count,
            _dptr(route_out), _dptr(indices), _dptr(weights)))

    def moe_forward_ep(self, hidden, router_fp16, top_k, intermediate, gate_up_local, down_local,
                       expert_begin, expert_count, group, stage_rows, out, indices=None,
                       weights=None):
        """The expert-parallel MoE op as one call: route rows go to every rank's staging
        buffer over peer mappings and the combine reads them there."""
        t, h = hidden.shape
        e = router_fp16.shape[0]
        self._check(lib().b2w4_moe_forward_ep(
            self.handle, _dptr(hidden), hidden.stride(0), t, h, _dptr(router_fp16), e, top_k,
            intermediate, gate_up_local.handle, down_local.handle, expert_begin, expert_count,
            C.byref(group), stage_rows, _dptr(out), out.stride(0),
            _dptr(indices) if indices is not None else None,
            _dptr(weights) if weights is not None else None))

    def moe_combine(self, route_out, top_k, indices, weights, out):
        t, h = out.shape
        self._check(lib().b2w4_moe_combine(self.handle, _dptr(route_out), t, h, top_k,
                                           _dptr(indices), _dptr(weights), _dptr(out),
                                           out.stride(0)))

    def select_routes(self, logits, top_k, indices, weights):
        t, e = logits.shape
        self._check(lib().b2w4_moe_select_routes(self.handle, _dptr(logits), t, e, top_k,
                                                 _dptr(indices), _dptr(weights)))
