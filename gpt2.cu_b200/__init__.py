"""ctypes binding of libgpt2_linear.so — the B200 (sm_100a) linear-layer GEMM path of gpt2.cu.

The library itself (C ABI: include/gpt2_linear.h) is the product; this module only loads it and
gives the tests and the benchmark a thin, typed way to call it with raw device pointers (for
example torch tensors' ``data_ptr()``). There is no fallback of any kind: if the shared library
is missing, import fails; if there is no sm_100 GPU, every compute call returns
``ERR_NO_DEVICE`` / ``ERR_NOT_INIT`` and the helpers here raise.

The directory name contains a dot, so import it through ``__graft_entry__.load_package()``
(which registers it as module ``gpt2cu_b200``).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libgpt2_linear.so")

OK = 0
ERR_NO_DEVICE = -1
ERR_BAD_ARG = -2
ERR_CUDA = -3
ERR_NOT_INIT = -4
ERR_TOO_LARGE = -5
ERR_SCHEDULE = -6
DEV_TIMEOUT = 1

MODE_TF32 = 0
MODE_TF32X3 = 1
EPI_GELU_DUAL = 1
AUX_NONE, AUX_ADD, AUX_GELU_GRAD = 0, 1, 2

OP_FORWARD = 0
OP_BACKWARD_INPUT = 1
OP_BACKWARD_WEIGHT = 2

DEP_NONE = 0
DEP_ROWBLOCK = 1
DEP_WHOLE_OP = 2
MAX_DEPS = 2

# every symbol include/gpt2_linear.h declares
EXPORTS = [
    "gpt2_linear_init", "gpt2_linear_shutdown", "gpt2_linear_version", "gpt2_linear_launch_count",
    "gpt2_linear_last_status",
    "gpt2_linear_forward", "gpt2_linear_backward_input", "gpt2_linear_backward_weight", "gpt2_linear_forward_xent",
    "gpt2_linear_forward_host", "gpt2_linear_backward_input_host", "gpt2_linear_backward_weight_host",
    "gpt2_linear_backward_weight_noalloc", "gpt2_linear_noalloc_last_status", "gpt2_linear_noalloc_debug_set_status",
    "gpt2_linear_forward_host_async", "gpt2_linear_backward_input_host_async",
    "gpt2_linear_backward_weight_host_async", "gpt2_linear_host_synchronize",
    "gpt2_schedule_create", "gpt2_schedule_destroy", "gpt2_schedule_validate", "gpt2_schedule_describe",
    "gpt2_megakernel_run", "gpt2_megakernel_status", "gpt2_schedule_debug_set_expected",
    "gpt2_schedule_profile", "gpt2_schedule_read_profile",
]
# every symbol include/gpt2_model.h declares
ATTENTION_EXPORTS = ["gpt2_attention_supported", "gpt2_attention_forward", "gpt2_attention_backward",
                     "gpt2_attention_status"]
ATT_FLASH, ATT_GEMM, ATT_SIMT = 0, 1, 2

MODEL_EXPORTS = [
    "gpt2_model_create", "gpt2_model_destroy", "gpt2_model_num_params", "gpt2_model_params", "gpt2_model_grads",
    "gpt2_model_param_offsets", "gpt2_model_set_params", "gpt2_model_get_params", "gpt2_model_get_grads",
    "gpt2_model_forward", "gpt2_model_backward", "gpt2_model_update", "gpt2_model_mean_loss",
    "gpt2_model_backward_head", "gpt2_model_backward_layer", "gpt2_model_backward_embedding",
    "gpt2_model_device_bytes", "gpt2_model_update_range", "gpt2_model_load_weights", "gpt2_model_dump_weights",
    "gpt2_model_save_checkpoint", "gpt2_model_load_checkpoint", "gpt2_model_forward_backward_graph",
    "gpt2_schedule_instructions", "gpt2_free_schedule", "gpt2_megakernel_step", "gpt2_megakernel_step_status",
    "gpt2_megakernel_step_info", "gpt2_megakernel_step_debug_set_expected",
    "gpt2_megakernel_step_profile", "gpt2_megakernel_step_read_profile",
]
STEP_WITH_UPDATE = 1
STEP_ATTENTION_IN_KERNEL = 2


class Opts(ctypes.Structure):
    """struct gpt2_linear_opts"""
    _fields_ = [
        ("mode", ctypes.c_int),
        ("flags", ctypes.c_uint),
        ("split_k", ctypes.c_int),
        ("deterministic", ctypes.c_int),
        ("out2", ctypes.c_void_p),
        ("force_simt", ctypes.c_int),
        ("cta_pair", ctypes.c_int),
        ("aux", ctypes.c_void_p),
        ("aux_op", ctypes.c_int),
        ("xent_lse", ctypes.c_void_p),
        ("xent_targets", ctypes.c_void_p),
        ("xent_vocab", ctypes.c_int),
        ("xent_scale", ctypes.c_float),
    ]


class Dep(ctypes.Structure):
    """struct gpt2l_dep"""
    _fields_ = [("producer", ctypes.c_int), ("kind", ctypes.c_int)]


class Op(ctypes.Structure):
    """struct gpt2l_op"""
    _fields_ = [
        ("kind", ctypes.c_int),
        ("layer", ctypes.c_int),
        ("B", ctypes.c_int), ("S", ctypes.c_int), ("K", ctypes.c_int), ("N", ctypes.c_int),
        ("out", ctypes.c_void_p),
        ("out_bias", ctypes.c_void_p),
        ("a", ctypes.c_void_p),
        ("b", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("opts", Opts),
        ("deps", Dep * MAX_DEPS),
    ]


class ModelConfig(ctypes.Structure):
    """struct gpt2_model_config"""
    _fields_ = [
        ("vocab_size", ctypes.c_int), ("padded_vocab_size", ctypes.c_int), ("n_layer", ctypes.c_int),
        ("n_head", ctypes.c_int), ("n_embd", ctypes.c_int), ("n_positions", ctypes.c_int),
    ]


class LinearError(RuntimeError):
    def __init__(self, fn, code):
        super().__init__(f"{fn} returned {code}")
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python gpt2.cu_b200/build.py` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    P, I, V = ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p
    OP = ctypes.POINTER(Opts)
    lib.gpt2_linear_init.argtypes = [I]
    lib.gpt2_linear_init.restype = I
    lib.gpt2_linear_shutdown.argtypes = []
    lib.gpt2_linear_shutdown.restype = None
    lib.gpt2_linear_version.restype = I
    lib.gpt2_linear_launch_count.restype = ctypes.c_longlong
    lib.gpt2_linear_last_status.argtypes = [ctypes.POINTER(I * 6)]
    lib.gpt2_linear_last_status.restype = I
    for name in ("gpt2_linear_forward", "gpt2_linear_forward_host"):
        f = getattr(lib, name)
        f.argtypes = [P, P, P, P, I, I, I, I, OP, V]
        f.restype = I
    for name in ("gpt2_linear_backward_input", "gpt2_linear_backward_input_host"):
        f = getattr(lib, name)
        f.argtypes = [P, P, P, I, I, I, I, OP, V]
        f.restype = I
    for name in ("gpt2_linear_backward_weight", "gpt2_linear_backward_weight_host",
                 "gpt2_linear_backward_weight_noalloc"):
        f = getattr(lib, name)
        f.argtypes = [P, P, P, P, I, I, I, I, OP, V]
        f.restype = I
    lib.gpt2_linear_forward_xent.argtypes = [P, P, P, P, P, P, I, I, I, I, I, OP, V]
    lib.gpt2_linear_forward_xent.restype = I
    lib.gpt2_linear_noalloc_last_status.argtypes = [ctypes.POINTER(I * 6)]
    lib.gpt2_linear_noalloc_last_status.restype = I
    lib.gpt2_linear_noalloc_debug_set_status.argtypes = [ctypes.POINTER(I * 6)]
    lib.gpt2_linear_noalloc_debug_set_status.restype = I
    lib.gpt2_linear_forward_host_async.argtypes = [P, P, P, P, I, I, I, I, OP]
    lib.gpt2_linear_forward_host_async.restype = I
    lib.gpt2_linear_backward_input_host_async.argtypes = [P, P, P, I, I, I, I, OP]
    lib.gpt2_linear_backward_input_host_async.restype = I
    lib.gpt2_linear_backward_weight_host_async.argtypes = [P, P, P, P, I, I, I, I, OP]
    lib.gpt2_linear_backward_weight_host_async.restype = I
    lib.gpt2_linear_host_synchronize.argtypes = []
    lib.gpt2_linear_host_synchronize.restype = I
    lib.gpt2_schedule_create.argtypes = [ctypes.POINTER(Op), I, ctypes.POINTER(I)]
    lib.gpt2_schedule_create.restype = V
    lib.gpt2_schedule_destroy.argtypes = [V]
    lib.gpt2_schedule_destroy.restype = None
    lib.gpt2_schedule_validate.argtypes = [ctypes.POINTER(Op), I, I]
    lib.gpt2_schedule_validate.restype = I
    lib.gpt2_schedule_describe.argtypes = [ctypes.POINTER(Op), I, I, ctypes.POINTER(I * 3)]
    lib.gpt2_schedule_describe.restype = I
    lib.gpt2_megakernel_run.argtypes = [V, V]
    lib.gpt2_megakernel_run.restype = I
    lib.gpt2_megakernel_status.argtypes = [V]
    lib.gpt2_megakernel_status.restype = I
    lib.gpt2_schedule_debug_set_expected.argtypes = [V, I, I, I, I]
    lib.gpt2_schedule_debug_set_expected.restype = I
    # ---- gpt2_model.h ----
    LL = ctypes.c_longlong
    F = ctypes.c_float
    lib.gpt2_model_create.argtypes = [ctypes.POINTER(ModelConfig), I, I, I, ctypes.POINTER(I)]
    lib.gpt2_model_create.restype = V
    lib.gpt2_model_destroy.argtypes = [V]
    lib.gpt2_model_destroy.restype = None
    lib.gpt2_model_num_params.argtypes = [V]
    lib.gpt2_model_num_params.restype = LL
    lib.gpt2_model_device_bytes.argtypes = [V]
    lib.gpt2_model_device_bytes.restype = LL
    lib.gpt2_model_params.argtypes = [V]
    lib.gpt2_model_params.restype = V
    lib.gpt2_model_grads.argtypes = [V]
    lib.gpt2_model_grads.restype = V
    lib.gpt2_model_param_offsets.argtypes = [V, ctypes.POINTER(LL), I]
    lib.gpt2_model_param_offsets.restype = I
    for name in ("gpt2_model_set_params", "gpt2_model_get_params", "gpt2_model_get_grads"):
        f = getattr(lib, name)
        f.argtypes = [V, P, LL]
        f.restype = I
    lib.gpt2_model_forward.argtypes = [V, P, P, V]
    lib.gpt2_model_forward.restype = I
    lib.gpt2_model_backward.argtypes = [V, V]
    lib.gpt2_model_backward.restype = I
    lib.gpt2_model_backward_head.argtypes = [V, V]
    lib.gpt2_model_backward_head.restype = I
    lib.gpt2_model_backward_layer.argtypes = [V, I, V]
    lib.gpt2_model_backward_layer.restype = I
    lib.gpt2_model_backward_embedding.argtypes = [V, V]
    lib.gpt2_model_backward_embedding.restype = I
    lib.gpt2_model_update.argtypes = [V, F, F, F, F, F, I, V]
    lib.gpt2_model_update.restype = I
    lib.gpt2_model_mean_loss.argtypes = [V, V]
    lib.gpt2_model_mean_loss.restype = F
    lib.gpt2_model_forward_backward_graph.argtypes = [V, P, P, V]
    lib.gpt2_model_forward_backward_graph.restype = I
    lib.gpt2_model_update_range.argtypes = [V, LL, LL, F, F, F, F, F, I, V]
    lib.gpt2_model_update_range.restype = I
    for name in ("gpt2_model_load_weights", "gpt2_model_dump_weights"):
        getattr(lib, name).argtypes = [V, ctypes.c_char_p]
        getattr(lib, name).restype = I
    lib.gpt2_model_save_checkpoint.argtypes = [V, ctypes.c_char_p, I]
    lib.gpt2_model_save_checkpoint.restype = I
    lib.gpt2_model_load_checkpoint.argtypes = [V, ctypes.c_char_p, ctypes.POINTER(I)]
    lib.gpt2_model_load_checkpoint.restype = I
    lib.gpt2_schedule_profile.argtypes = [V, I]
    lib.gpt2_schedule_profile.restype = I
    lib.gpt2_schedule_read_profile.argtypes = [V, P, LL]
    lib.gpt2_schedule_read_profile.restype = LL
    lib.gpt2_schedule_instructions.argtypes = [V, P, P, ctypes.c_uint, ctypes.POINTER(I)]
    lib.gpt2_schedule_instructions.restype = V
    lib.gpt2_free_schedule.argtypes = [V]
    lib.gpt2_free_schedule.restype = None
    lib.gpt2_megakernel_step.argtypes = [V, F, F, F, F, F, I, V]
    lib.gpt2_megakernel_step.restype = I
    lib.gpt2_megakernel_step_status.argtypes = [V]
    lib.gpt2_megakernel_step_status.restype = I
    lib.gpt2_megakernel_step_info.argtypes = [V, ctypes.POINTER(I * 3)]
    lib.gpt2_megakernel_step_info.restype = I
    lib.gpt2_megakernel_step_profile.argtypes = [V, I]
    lib.gpt2_megakernel_step_profile.restype = I
    lib.gpt2_megakernel_step_read_profile.argtypes = [V, I, P, LL]
    lib.gpt2_megakernel_step_read_profile.restype = LL
    lib.gpt2_megakernel_step_debug_set_expected.argtypes = [V, I, I, I, I, I]
    lib.gpt2_megakernel_step_debug_set_expected.restype = I
    # ---- gpt2_attention.h ----
    lib.gpt2_attention_supported.argtypes = [I, I, I, I]
    lib.gpt2_attention_supported.restype = I
    lib.gpt2_attention_forward.argtypes = [P, P, P, P, I, I, I, I, I, I, V]
    lib.gpt2_attention_forward.restype = I
    lib.gpt2_attention_backward.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, V]
    lib.gpt2_attention_backward.restype = I
    lib.gpt2_attention_status.restype = I
    return lib


lib = _load()


def check(fn, code):
    if code != 0:
        raise LinearError(fn, code)


def init(device=0):
    """gpt2_linear_init; raises when there is no sm_100 device (no fallback exists)."""
    check("gpt2_linear_init", lib.gpt2_linear_init(device))


def make_opts(mode=MODE_TF32, flags=0, split_k=0, deterministic=0, out2=None, force_simt=0, cta_pair=0, aux=None,
              aux_op=0, xent_lse=None, xent_targets=None, xent_vocab=0, xent_scale=0.0):
    return Opts(mode, flags, split_k, deterministic, out2, force_simt, cta_pair, _p(aux), aux_op, _p(xent_lse),
                _p(xent_targets), xent_vocab, xent_scale)


def _p(t):
    """device (or host) pointer of a torch tensor / numpy array / int / None"""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def forward(out, x, w, b, B, S, K, N, opts=None, stream=None, host=False):
    fn = lib.gpt2_linear_forward_host if host else lib.gpt2_linear_forward
    return fn(_p(out), _p(x), _p(w), _p(b), B, S, K, N, ctypes.byref(opts) if opts else None, stream)


def forward_xent(logits, losses, lse, x, w, targets, B, S, K, N, V, opts=None, stream=None):
    """gpt2_linear_forward_xent: lm_head forward with softmax statistics and the cross-entropy loss"""
    return lib.gpt2_linear_forward_xent(_p(logits), _p(losses), _p(lse), _p(x), _p(w), _p(targets), B, S, K, N, V,
                                        ctypes.byref(opts) if opts else None, stream)


def backward_input(g_in, g_out, w, B, S, K, N, opts=None, stream=None, host=False):
    fn = lib.gpt2_linear_backward_input_host if host else lib.gpt2_linear_backward_input
    return fn(_p(g_in), _p(g_out), _p(w), B, S, K, N, ctypes.byref(opts) if opts else None, stream)


def backward_weight(g_w, g_b, g_out, x, B, S, K, N, opts=None, stream=None, host=False):
    fn = lib.gpt2_linear_backward_weight_host if host else lib.gpt2_linear_backward_weight
    return fn(_p(g_w), _p(g_b), _p(g_out), _p(x), B, S, K, N, ctypes.byref(opts) if opts else None, stream)


def forward_host_async(out, x, w, b, B, S, K, N, opts=None):
    return lib.gpt2_linear_forward_host_async(_p(out), _p(x), _p(w), _p(b), B, S, K, N,
                                              ctypes.byref(opts) if opts else None)


def backward_input_host_async(g_in, g_out, w, B, S, K, N, opts=None):
    return lib.gpt2_linear_backward_input_host_async(_p(g_in), _p(g_out), _p(w), B, S, K, N,
                                                     ctypes.byref(opts) if opts else None)


def backward_weight_host_async(g_w, g_b, g_out, x, B, S, K, N, opts=None):
    return lib.gpt2_linear_backward_weight_host_async(_p(g_w), _p(g_b), _p(g_out), _p(x), B, S, K, N,
                                                      ctypes.byref(opts) if opts else None)


def host_synchronize():
    return lib.gpt2_linear_host_synchronize()


def attention_forward(out, lse, probs, qkv, B, T, NH, C, impl=ATT_FLASH, mode=MODE_TF32, stream=None):
    """gpt2_attention_forward (include/gpt2_attention.h)"""
    return lib.gpt2_attention_forward(_p(out), _p(lse), _p(probs), _p(qkv), B, T, NH, C, impl, mode, stream)


def attention_backward(g_qkv, g_out, qkv, out, lse, probs, row_scratch, tt_scratch, B, T, C, NH, impl=ATT_FLASH,
                       mode=MODE_TF32, stream=None):
    """gpt2_attention_backward (include/gpt2_attention.h)"""
    return lib.gpt2_attention_backward(_p(g_qkv), _p(g_out), _p(qkv), _p(out), _p(lse), _p(probs), _p(row_scratch),
                                       _p(tt_scratch), B, T, C, NH, impl, mode, stream)


def backward_weight_noalloc(g_w, g_b, g_out, x, B, S, K, N, opts=None, stream=None):
    """gpt2_linear_backward_weight_noalloc: deterministic split-K weight gradient whose workspace is a
    fixed array in the library image (for callers that must not allocate device memory)."""
    return lib.gpt2_linear_backward_weight_noalloc(_p(g_w), _p(g_b), _p(g_out), _p(x), B, S, K, N,
                                                   ctypes.byref(opts) if opts else None, stream)


def noalloc_last_status():
    """gpt2_linear_noalloc_last_status: (status word, record) of the no-allocation path; clears a non-zero record."""
    rec = (ctypes.c_int * 6)()
    st = lib.gpt2_linear_noalloc_last_status(ctypes.byref(rec))
    return st, list(rec)


def noalloc_debug_set_status(rec):
    arr = (ctypes.c_int * 6)(*rec)
    return lib.gpt2_linear_noalloc_debug_set_status(ctypes.byref(arr))


def last_status():
    rec = (ctypes.c_int * 6)()
    st = lib.gpt2_linear_last_status(ctypes.byref(rec))
    return st, list(rec)


def make_op(kind, B, S, K, N, out, a, b, bias=None, out_bias=None, opts=None, deps=(), layer=0):
    """One entry of a megakernel schedule. deps = [(producer_index, DEP_*), ...]"""
    op = Op()
    op.kind, op.layer, op.B, op.S, op.K, op.N = kind, layer, B, S, K, N
    op.out, op.out_bias, op.a, op.b, op.bias = _p(out), _p(out_bias), _p(a), _p(b), _p(bias)
    op.opts = opts if opts is not None else make_opts()
    for i, (prod, kind_) in enumerate(deps):
        op.deps[i].producer = prod
        op.deps[i].kind = kind_
    return op


class Schedule:
    """Owns a gpt2l_schedule (device op array, counters) built from a list of Op."""

    def __init__(self, ops):
        self.n = len(ops)
        self.arr = (Op * self.n)(*ops)
        err = ctypes.c_int(0)
        self.handle = lib.gpt2_schedule_create(self.arr, self.n, ctypes.byref(err))
        if not self.handle:
            raise LinearError("gpt2_schedule_create", err.value)

    def run(self, stream=None):
        return lib.gpt2_megakernel_run(self.handle, stream)

    def status(self):
        return lib.gpt2_megakernel_status(self.handle)

    def debug_set_expected(self, op, dep, expected, wait_limit_ms=0):
        return lib.gpt2_schedule_debug_set_expected(self.handle, op, dep, expected, wait_limit_ms)

    def close(self):
        if self.handle:
            lib.gpt2_schedule_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def validate_schedule(ops, grid):
    arr = (Op * len(ops))(*ops)
    return lib.gpt2_schedule_validate(arr, len(ops), grid)


def describe_schedule(ops, num_sms):
    arr = (Op * len(ops))(*ops)
    counts = (ctypes.c_int * 3)()
    code = lib.gpt2_schedule_describe(arr, len(ops), num_sms, ctypes.byref(counts))
    return code, list(counts)


class Model:
    """Owns a gpt2_model (include/gpt2_model.h): GPT-2 training step around the GEMM path."""

    def __init__(self, vocab_size, padded_vocab_size, n_layer, n_head, n_embd, n_positions, B, T, mode=MODE_TF32):
        self.cfg = ModelConfig(vocab_size, padded_vocab_size, n_layer, n_head, n_embd, n_positions)
        self.B, self.T = B, T
        err = ctypes.c_int(0)
        self.handle = lib.gpt2_model_create(ctypes.byref(self.cfg), B, T, mode, ctypes.byref(err))
        if not self.handle:
            raise LinearError("gpt2_model_create", err.value)
        self.num_params = lib.gpt2_model_num_params(self.handle)

    def offsets(self):
        n = 4 + 12 * self.cfg.n_layer
        arr = (ctypes.c_longlong * n)()
        got = lib.gpt2_model_param_offsets(self.handle, arr, n)
        if got != n:
            raise LinearError("gpt2_model_param_offsets", got)
        return list(arr)

    def set_params(self, host):
        check("gpt2_model_set_params", lib.gpt2_model_set_params(self.handle, _p(host), host.size))

    def get_params(self, host):
        check("gpt2_model_get_params", lib.gpt2_model_get_params(self.handle, _p(host), host.size))

    def get_grads(self, host):
        check("gpt2_model_get_grads", lib.gpt2_model_get_grads(self.handle, _p(host), host.size))

    def params_ptr(self):
        return lib.gpt2_model_params(self.handle)

    def grads_ptr(self):
        return lib.gpt2_model_grads(self.handle)

    def forward(self, tokens, targets, stream=None):
        return lib.gpt2_model_forward(self.handle, _p(tokens), _p(targets), stream)

    def backward(self, stream=None):
        return lib.gpt2_model_backward(self.handle, stream)

    def forward_backward_graph(self, tokens, targets, stream=None):
        return lib.gpt2_model_forward_backward_graph(self.handle, _p(tokens), _p(targets), stream)

    def backward_head(self, stream=None):
        return lib.gpt2_model_backward_head(self.handle, stream)

    def backward_layer(self, l, stream=None):
        return lib.gpt2_model_backward_layer(self.handle, l, stream)

    def backward_embedding(self, stream=None):
        return lib.gpt2_model_backward_embedding(self.handle, stream)

    def update(self, lr, beta1, beta2, eps, weight_decay, t, stream=None):
        return lib.gpt2_model_update(self.handle, lr, beta1, beta2, eps, weight_decay, t, stream)

    def update_range(self, first, count, lr, beta1, beta2, eps, weight_decay, t, stream=None):
        return lib.gpt2_model_update_range(self.handle, first, count, lr, beta1, beta2, eps, weight_decay, t, stream)

    def mean_loss(self, stream=None):
        return lib.gpt2_model_mean_loss(self.handle, stream)

    def load_weights(self, path):
        check("gpt2_model_load_weights", lib.gpt2_model_load_weights(self.handle, os.fsencode(path)))

    def dump_weights(self, path):
        check("gpt2_model_dump_weights", lib.gpt2_model_dump_weights(self.handle, os.fsencode(path)))

    def save_checkpoint(self, path, step):
        check("gpt2_model_save_checkpoint", lib.gpt2_model_save_checkpoint(self.handle, os.fsencode(path), step))

    def load_checkpoint(self, path):
        step = ctypes.c_int(-1)
        check("gpt2_model_load_checkpoint",
              lib.gpt2_model_load_checkpoint(self.handle, os.fsencode(path), ctypes.byref(step)))
        return step.value

    def device_bytes(self):
        return lib.gpt2_model_device_bytes(self.handle)

    def close(self):
        if self.handle:
            lib.gpt2_model_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Step:
    """Owns a gpt2l_step (include/gpt2_model.h): one training step of a Model as a schedule of the persistent
    kernel. tokens / targets are device int32 tensors that must outlive the object."""

    def __init__(self, model, tokens, targets, with_update=True, attention_in_kernel=False):
        self.model, self.tokens, self.targets = model, tokens, targets
        flags = (STEP_WITH_UPDATE if with_update else 0) | (STEP_ATTENTION_IN_KERNEL if attention_in_kernel else 0)
        err = ctypes.c_int(0)
        self.handle = lib.gpt2_schedule_instructions(model.handle, _p(tokens), _p(targets), flags, ctypes.byref(err))
        if not self.handle:
            raise LinearError("gpt2_schedule_instructions", err.value)

    def run(self, lr=0.0, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, t=1, stream=None):
        return lib.gpt2_megakernel_step(self.handle, lr, beta1, beta2, eps, weight_decay, t, stream)

    def status(self):
        return lib.gpt2_megakernel_step_status(self.handle)

    def info(self):
        out = (ctypes.c_int * 3)()
        check("gpt2_megakernel_step_info", lib.gpt2_megakernel_step_info(self.handle, ctypes.byref(out)))
        return {"ops": out[0], "launches": out[1], "tiles": out[2]}

    def profile(self, enable=True):
        check("gpt2_megakernel_step_profile", lib.gpt2_megakernel_step_profile(self.handle, 1 if enable else 0))

    def read_profile(self, piece, max_tiles=1 << 22):
        """numpy int64 array [tiles][4] = (op index, op kind, start ns, duration ns, SM) -> columns op, kind, start, ns, sm"""
        import numpy as np
        buf = np.zeros((max_tiles, 4), np.int64)
        n = lib.gpt2_megakernel_step_read_profile(self.handle, piece, buf.ctypes.data, max_tiles)
        if n < 0:
            return None
        buf = buf[:n]
        out = np.zeros((n, 5), np.int64)
        out[:, 0] = buf[:, 0] & 0xffffffff
        out[:, 1] = buf[:, 0] >> 32
        out[:, 2:] = buf[:, 1:]
        return out

    def debug_set_expected(self, piece, op, dep, expected, wait_limit_ms=0):
        return lib.gpt2_megakernel_step_debug_set_expected(self.handle, piece, op, dep, expected, wait_limit_ms)

    def close(self):
        if self.handle:
            lib.gpt2_free_schedule(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
