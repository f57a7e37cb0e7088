"""Host-side mirror of the reference's ``sparseconvnet.SCN`` extension module.

Same names, argument order and ownership rules as the functions bound in the reference's
``sparseconvnet/SCN/pybind.cpp:201-237`` (prototypes in ``sparseconvnet/SCN/sparseconvnet.h``)
for the inference path: the caller passes an empty output tensor, the callee sizes and
fills it; an absent bias is a 0-element tensor; spatial sizes are CPU LongTensors;
convolutions return their multiply-add count as a float.

Every function forwards to the C-ABI library (``include/scn_b200.h``) with raw device
pointers and torch's current CUDA stream.  Feature tensors must be CUDA float32: there is
no CPU path.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import check, lib, sizes

class DeferredCount(object):
    """Multiply-add count of a convolution whose rule totals were still on their way to the host
    when the operator returned (``scn_set_deferred_counts`` in ``include/scn_b200.h``).  Acts as
    the number: ``float(x)``, ``x + y``, ``x * y`` wait for that one copy and give the count the
    reference's operator would have returned (CPU/Convolution.cpp:141)."""
    __slots__ = ("_ticket", "_factor", "_value")

    def __init__(self, ticket, factor):
        self._ticket, self._factor, self._value = ticket, factor, None

    def resolve(self):
        if self._value is None:
            total = C.c_int64()
            check(lib.scn_count_ticket_total(self._ticket, C.byref(total)))
            self._value = float(total.value) * self._factor
            lib.scn_count_ticket_release(self._ticket)
            self._ticket = None
        return self._value

    def __del__(self):
        if getattr(self, "_ticket", None) is not None and lib is not None:
            lib.scn_count_ticket_release(self._ticket)
            self._ticket = None

    __float__ = resolve

    def __int__(self):
        return int(self.resolve())

    def __add__(self, other):
        return self.resolve() + other

    __radd__ = __add__

    def __mul__(self, other):
        return self.resolve() * other

    __rmul__ = __mul__

    def __truediv__(self, other):
        return self.resolve() / other

    def __rtruediv__(self, other):
        return other / self.resolve()

    def __sub__(self, other):
        return self.resolve() - other

    def __rsub__(self, other):
        return other - self.resolve()

    def __eq__(self, other):
        return self.resolve() == other

    def __lt__(self, other):
        return self.resolve() < other

    def __gt__(self, other):
        return self.resolve() > other

    __hash__ = None

    def __repr__(self):
        return "DeferredCount(%r)" % (self._value if self._value is not None else "pending")


class _FlopCounter(object):
    """``forward_pass_multiplyAdd_count`` of the package: counts still in flight are kept aside
    and folded in when the number is read (or when about two forward passes' worth have piled up)."""

    def __init__(self):
        self.base, self.pending = 0, []

    def add(self, macs):
        if isinstance(macs, DeferredCount):
            self.pending.append(macs)
            if len(self.pending) > 96:
                # the oldest ones landed a forward pass ago: folding them waits for nothing and gives
                # their tickets (pinned memory, an event) back to the library's pool
                old, self.pending = self.pending[:48], self.pending[48:]
                for p in old:
                    self.base += p.resolve()
        else:
            self.base += macs

    def fold(self):
        pending, self.pending = self.pending, []
        for p in pending:
            self.base += p.resolve()

    def value(self):
        self.fold()
        return self.base

    def reset(self, value=0):
        self.base, self.pending = value, []


flop_counter = _FlopCounter()
check(lib.scn_set_deferred_counts(1))


def _macs_result(m, macs):
    if macs.value >= 0:
        return macs.value
    ticket = C.c_void_p()
    check(lib.scn_md_take_count_ticket(m._h, C.byref(ticket)))
    if not ticket.value:
        raise RuntimeError("count pending but no ticket")
    return DeferredCount(ticket.value, -macs.value)


# scn_last_conv_kernel() -> name (enum scn_conv_kernel of include/scn_b200.h)
_KERNEL_NAMES = ("k_conv_simt", "k_conv_tc", "k_conv_tma", "k_conv_pipe_mma", "k_conv_rows", "k_conv_wide")

PRECISION_FP32, PRECISION_TF32, PRECISION_BF16, PRECISION_TF32X3 = 0, 1, 2, 3
_precision = PRECISION_FP32


def set_precision(p):
    """Arithmetic of the convolution kernels: 'fp32' (default; fp32 FMA), 'tf32x3' (tensor-core
    tiles over the hi/lo split of both operands: fp32-class accuracy), 'tf32' or 'bf16'
    (single-pass tensor-core tiles, fp32 accumulation)."""
    global _precision
    table = {"fp32": 0, "tf32": 1, "bf16": 2, "tf32x3": 3, 0: 0, 1: 1, 2: 2, 3: 3}
    if p not in table:
        raise ValueError("precision must be 'fp32', 'tf32x3', 'tf32' or 'bf16'")
    _precision = table[p]


def get_precision():
    return ("fp32", "tf32", "bf16", "tf32x3")[_precision]


_backward_precision = PRECISION_FP32


def set_backward_precision(p):
    """Arithmetic of the input-gradient pass of the convolutions' backward (the forward kernels on
    the opposite rulebook table): 'fp32' (default) or 'tf32x3' keep fp32-class gradients, 'tf32' /
    'bf16' are single-pass.  Weight and bias gradients are always reduced in fp32."""
    global _backward_precision
    table = {"fp32": 0, "tf32": 1, "bf16": 2, "tf32x3": 3, 0: 0, 1: 1, 2: 2, 3: 3}
    if p not in table:
        raise ValueError("precision must be 'fp32', 'tf32x3', 'tf32' or 'bf16'")
    check(lib.scn_set_backward_precision(table[p]))
    _backward_precision = table[p]


def get_backward_precision():
    return ("fp32", "tf32", "bf16", "tf32x3")[_backward_precision]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) if torch is not None else None


def _stream():
    """The current CUDA stream of the current device as a handle for the C ABI."""
    if _raw_stream is not None:  # the same handle without building a Stream object (8 us -> 0.5 us per call)
        return C.c_void_p(_raw_stream(torch.cuda.current_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on_device(object):
    """``torch.cuda.device(dev)`` for the common case that `dev` is already the current device: then it
    costs one query instead of a device switch there and back (about 10 us per operator call)."""
    __slots__ = ("idx", "prev")

    def __init__(self, dev):
        self.idx = dev.index if isinstance(dev, torch.device) else (None if dev is None else int(dev))
        self.prev = -1

    def __enter__(self):
        if self.idx is not None:
            cur = torch.cuda.current_device()
            if cur != self.idx:
                self.prev = cur
                torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
            self.prev = -1


class Profile(object):
    """Optional per-operator timing: inside ``with SCN.Profile() as p`` every operator call
    records a pair of CUDA events on the current stream around its kernels, plus the sizes
    needed to turn the time into algorithmic bytes and FLOPs.  ``p.rows()`` (after a
    synchronize) lists dicts with ``kind``, ``ms`` and those sizes.  Off by default."""
    active = None

    def __enter__(self):
        self.records = []
        Profile.active = self
        return self

    def __exit__(self, *exc):
        Profile.active = None

    def rows(self):
        torch.cuda.synchronize()
        return [dict(info, kind=kind, ms=a.elapsed_time(b)) for kind, info, a, b in self.records]


class _timed(object):
    def __init__(self, kind, info):
        self.kind, self.info = kind, info

    def __enter__(self):
        p = Profile.active
        if p is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.b = torch.cuda.Event(enable_timing=True)
            self.a.record()
        return self.info

    def __exit__(self, *exc):
        p = Profile.active
        if p is not None and exc[0] is None:
            self.b.record()
            p.records.append((self.kind, self.info, self.a, self.b))


_token_counter = [0]


def new_weight_token():
    """A fresh non-zero token for scn_set_weight_token (see include/scn_b200.h)."""
    _token_counter[0] += 1
    return _token_counter[0]


class weight_token(object):
    """``with SCN.weight_token(t):`` -- convolution calls inside keep / reuse their prepared weight
    images under token `t` (0: no caching)."""

    def __init__(self, token):
        self.token = int(token)

    def __enter__(self):
        if self.token:
            lib.scn_set_weight_token(self.token)

    def __exit__(self, *exc):
        if self.token:
            lib.scn_set_weight_token(0)


def release_weight_token(token):
    if token and torch is not None and lib is not None:
        try:
            lib.scn_release_weight_token(int(token), _stream() if torch.cuda.is_available() else None)
        except Exception:  # interpreter shutdown: the process's memory goes with it
            pass


def launch_count():
    """Kernels launched by the library in this process so far."""
    return lib.scn_launch_count()


def host_wait_count():
    """Times the library has made the calling thread wait for the GPU in this process so far."""
    return lib.scn_host_wait_count()


def _features(t, name):
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor: sparseconvnet_b200 has no CPU path" % name)
    if t.dtype != torch.float32:
        raise RuntimeError("%s must be float32, got %s" % (name, t.dtype))
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    return t


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None and t.numel() else C.c_void_p(0)


def _optional(t, like, name):
    """0-element tensor means 'absent' (reference: utils.py:21-22, bias.numel() tests)."""
    if t is None or t.numel() == 0:
        return None
    t = _features(t.detach(), name)
    if t.device != like.device:
        raise RuntimeError("%s is on %s, features on %s" % (name, t.device, like.device))
    return t


class _Metadata(object):
    """Counterpart of the reference's ``Metadata<D>`` Python object (pybind.cpp:12-33): owns
    the GPU site hash of every spatial scale and the rulebook cache."""
    dimension = 0

    def __init__(self):
        self._h = C.c_void_p()
        check(lib.scn_md_create(self.dimension, C.byref(self._h)))
        self.device = None
        self.chain_looked_for = False  # containers.Sequential: has a container looked for an encoder to prefetch?
        self.chain_started = False     # ... and started one (SCN.strided_chain_start)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:
            try:
                lib.scn_md_destroy(h)
            except Exception:
                pass

    def clear(self):
        check(lib.scn_md_clear(self._h, _stream()))

    def poll_errors(self):
        """Waits for the current stream and raises if a kernel flagged a problem."""
        dev = self.device if self.device is not None else torch.device("cuda")
        with _on_device(dev):
            check(lib.scn_md_poll_errors(self._h, _stream()))

    def getNActive(self, spatial_size):
        n = C.c_int64()
        check(lib.scn_md_n_active(self._h, sizes(spatial_size), C.byref(n)))
        return n.value

    def getBatchSize(self, spatial_size):
        n = C.c_int64()
        check(lib.scn_md_batch_size(self._h, sizes(spatial_size), C.byref(n)))
        return n.value

    def getSpatialLocations(self, spatial_size, device="cpu"):
        """LongTensor [nActive, D+1]: coordinates then batch index (Metadata.cpp:149-170).
        Computed on the GPU; returned on the CPU like the reference unless ``device`` says
        otherwise."""
        n = self.getNActive(spatial_size)
        dev = self.device if self.device is not None else torch.device("cuda")
        out = torch.zeros(n, self.dimension + 1, dtype=torch.int64, device=dev)
        if n:
            with _on_device(dev):
                check(lib.scn_md_spatial_locations(self._h, sizes(spatial_size), _ptr(out), _stream()))
        return out.to(device)

    # ---- extensions used by tests and tools (no counterpart in the reference's bindings) ----
    def rulebook(self, kind, a, b, c=None):
        """Reads a built rulebook back as the reference stores it: a list with one int32
        tensor [n_rules, 2] of (input_row, output_row) per filter offset."""
        dev = self.device if self.device is not None else torch.device("cuda")
        n_off = C.c_int64()
        counts = (C.c_int64 * 4096)()
        sc = sizes(c) if c is not None else None
        with _on_device(dev):
            check(lib.scn_md_rulebook_export(self._h, kind, sizes(a), sizes(b), sc, C.byref(n_off), counts,
                                             None, _stream()))
            k = n_off.value
            cnt = [counts[i] for i in range(k)]
            pairs = torch.empty(2 * sum(cnt), dtype=torch.int32, device=dev)
            check(lib.scn_md_rulebook_export(self._h, kind, sizes(a), sizes(b), sc, C.byref(n_off), counts,
                                             _ptr(pairs), _stream()))
        pairs = pairs.view(-1, 2)
        out, pos = [], 0
        for n in cnt:
            out.append(pairs[pos:pos + n])
            pos += n
        return out

    def _unsupported(self, *a, **k):
        raise NotImplementedError("outside the inference path implemented by sparseconvnet_b200")

    setInputSpatialSize = batchAddSample = setInputSpatialLocation = setInputSpatialLocations = _unsupported
    createMetadataForDenseToSparse = sparsifyMetadata = appendMetadata = sparsifyCompare = _unsupported
    addSampleFromThresholdedTensor = generateRuleBooks3s2 = generateRuleBooks2s2 = _unsupported
    compareSparseHelper = copyFeaturesHelper = _unsupported


def _make_metadata_class(d):
    return type("Metadata_%d" % d, (_Metadata,), {"dimension": d})


Metadata_1, Metadata_2, Metadata_3, Metadata_4, Metadata_5, Metadata_6 = (
    _make_metadata_class(d) for d in range(1, 7))


def n_rulebook_bits():
    return 32


def is_cuda_build():
    return True


# ---------------------------------------------------------------------------------------------
# operators
# ---------------------------------------------------------------------------------------------

def InputLayer_updateOutput(m, spatial_size, input_coords, input_features, output_features,
                            batch_size, mode):
    """sparseconvnet.h:163-167.  ``input_coords`` may be a CPU or CUDA LongTensor."""
    f = _features(input_features, "input_features")
    if input_coords.dtype != torch.int64 or input_coords.dim() != 2:
        raise RuntimeError("input_coords must be a 2-d LongTensor")
    if input_coords.size(0) != f.size(0):
        raise RuntimeError("input_coords and input_features disagree on the row count")
    coords = input_coords.contiguous()
    if coords.is_cuda and coords.device != f.device:
        coords = coords.to(f.device)
    m.device = f.device
    m.chain_looked_for = False  # a new input: the containers may look for an encoder to prefetch again
    m.chain_started = False
    m.n_input_rows, m.bl_shape = coords.size(0), None
    n_active = C.c_int64()
    with _on_device(f.device):
        with _timed("input_hash", dict(rows=coords.size(0), cols=coords.size(1), mode=int(mode))) as info:
            check(lib.scn_md_input_layer(m._h, sizes(spatial_size), _ptr(coords), int(coords.is_cuda),
                                         coords.size(0), coords.size(1), int(batch_size), int(mode),
                                         _stream(), C.byref(n_active)))
            info["sites"] = n_active.value
        output_features.resize_(n_active.value, f.size(1))
        with _timed("input_features", dict(rows=coords.size(0), sites=n_active.value, planes=f.size(1))):
            check(lib.scn_input_layer_forward(m._h, _ptr(f), f.size(0), _ptr(output_features), n_active.value,
                                              f.size(1), _stream()))


def BLInputLayer_updateOutput(m, spatial_size, input_coords, input_features, output_features, mode):
    """sparseconvnet.h (BLInputLayer_updateOutput), CPU/IOLayers.cpp:139-163.  ``input_coords``:
    LongTensor [batch, length, dimension] on the CPU or the GPU, -1 marks an empty slot;
    ``input_features``: [batch, length, planes]."""
    f = _features(input_features, "input_features")
    if input_coords.dtype != torch.int64 or input_coords.dim() != 3:
        raise RuntimeError("input_coords must be a 3-d LongTensor [batch, length, dimension]")
    if f.dim() != 3 or tuple(input_coords.shape[:2]) != tuple(f.shape[:2]):
        raise RuntimeError("input_coords and input_features disagree on batch x length")
    coords = input_coords.contiguous()
    if coords.is_cuda and coords.device != f.device:
        coords = coords.to(f.device)
    m.device = f.device
    m.chain_looked_for = False  # a new input: the containers may look for an encoder to prefetch again
    m.bl_shape, m.n_input_rows = (f.size(0), f.size(1)), f.size(0) * f.size(1)
    n_active = C.c_int64()
    with _on_device(f.device):
        with _timed("input_hash", dict(rows=f.size(0) * f.size(1), cols=coords.size(2), mode=int(mode))) as info:
            check(lib.scn_md_bl_input_layer(m._h, sizes(spatial_size), _ptr(coords), int(coords.is_cuda),
                                            f.size(0), f.size(1), int(mode), _stream(), C.byref(n_active)))
            info["sites"] = n_active.value
        output_features.resize_(n_active.value, f.size(2))
        with _timed("input_features", dict(rows=f.size(0) * f.size(1), sites=n_active.value, planes=f.size(2))):
            check(lib.scn_input_layer_forward(m._h, _ptr(f), f.size(0) * f.size(1), _ptr(output_features),
                                              n_active.value, f.size(2), _stream()))


def _output_layer(m, input_features, output_features, shape):
    f = _features(input_features, "input_features")
    n_points = 1
    for d in shape[:-1]:
        n_points *= d
    output_features.resize_(*shape)
    with _on_device(f.device):
        with _timed("output_features", dict(rows=n_points, sites=f.size(0), planes=f.size(1))):
            check(lib.scn_output_layer_forward(m._h, _ptr(f), f.size(0), _ptr(output_features), n_points,
                                               f.size(1), _stream()))


def OutputLayer_updateOutput(m, input_features, output_features):
    """CPU/IOLayers.cpp:95-114: [n_active, planes] -> [n_points, planes] of the InputLayer call."""
    if getattr(m, "n_input_rows", None) is None:
        raise RuntimeError("OutputLayer needs a metadata made by InputLayer")
    _output_layer(m, input_features, output_features, (m.n_input_rows, input_features.size(1)))


def BLOutputLayer_updateOutput(m, input_features, output_features):
    """CPU/IOLayers.cpp:197-215: [n_active, planes] -> [batch, length, planes] of the BLInputLayer call."""
    if getattr(m, "bl_shape", None) is None:
        raise RuntimeError("BLOutputLayer needs a metadata made by BLInputLayer")
    _output_layer(m, input_features, output_features, m.bl_shape + (input_features.size(1),))


def _conv_args(input_features, weight, bias):
    f = _features(input_features, "input_features")
    w = _features(weight.detach(), "weight")
    if w.dim() != 4:
        raise RuntimeError("weight must be [filter_volume, groups, nIn/groups, nOut/groups]")
    if w.device != f.device:
        raise RuntimeError("weight is on %s, features on %s" % (w.device, f.device))
    groups, cin, cout = w.size(1), w.size(2), w.size(3)
    if f.numel() and f.size(1) != groups * cin:
        raise RuntimeError("features have %d planes, weight expects %d" % (f.size(1), groups * cin))
    b = _optional(bias, f, "bias")
    return f, w, b, groups, cin, cout


def _epilogue_args(epilogue, f, planes):
    """(scale ptr, shift ptr, leakiness) of an optional fused BatchNorm: `epilogue` = (scale [planes],
    shift [planes], leakiness) as made by batchnorm_fold."""
    scale, shift, leak = epilogue
    for t in (scale, shift):
        if not t.is_cuda or t.dtype != torch.float32 or t.numel() != planes or t.device != f.device:
            raise RuntimeError("fused BatchNorm: scale / shift must be CUDA float32 [%d] on %s" % (planes, f.device))
    return _ptr(scale), _ptr(shift), float(leak)


def batchnorm_fold(running_mean, running_var, weight, bias, eps):
    """scale = weight / sqrt(running_var + eps), shift = bias - running_mean * scale of an eval-mode
    BatchNormalization (CPU/BatchNormalization.cpp:41-46), computed on the device with the roundings
    of the stand-alone operator.  Returns (scale, shift)."""
    c = running_mean.numel()
    scale, shift = running_mean.new_empty(c), running_mean.new_empty(c)
    w = _optional(weight, running_mean, "weight")
    b = _optional(bias, running_mean, "bias")
    with _on_device(running_mean.device):
        check(lib.scn_batchnorm_fold(_ptr(running_mean), _ptr(running_var), _ptr(w), _ptr(b), float(eps), c,
                                     _ptr(scale), _ptr(shift), _stream()))
    return scale, shift


def SubmanifoldConvolution_updateOutput(inputSize, filterSize, m, input_features, output_features,
                                        weight, bias, epilogue=None):
    """sparseconvnet.h:101-104.  `epilogue` (not in the reference): see batchnorm_fold."""
    f, w, b, groups, cin, cout = _conv_args(input_features, weight, bias)
    macs = C.c_double()
    with _on_device(f.device):
        n = m.getNActive(inputSize)
        if f.size(0) != n:
            raise RuntimeError("features have %d rows, metadata has %d active sites" % (f.size(0), n))
        output_features.resize_(n, groups * cout)
        if Profile.active is None:  # the convolution entry finds or builds the rulebook itself
            if epilogue is None:
                check(lib.scn_submanifold_convolution_forward(
                    m._h, sizes(inputSize), sizes(filterSize), _ptr(f), _ptr(output_features), _ptr(w), _ptr(b),
                    groups * cin, groups * cout, groups, _precision, _stream(), C.byref(macs)))
            else:
                sc, sh, leak = _epilogue_args(epilogue, f, groups * cout)
                check(lib.scn_submanifold_convolution_bn_forward(
                    m._h, sizes(inputSize), sizes(filterSize), _ptr(f), _ptr(output_features), _ptr(w), _ptr(b),
                    sc, sh, leak, groups * cin, groups * cout, groups, _precision, _stream(), C.byref(macs)))
            return _macs_result(m, macs)
        # profiled: the rulebook call on its own, so that its time and bytes are not the convolution's
        with _timed("rules_submanifold", dict(sites=n, offsets=w.size(0), dim=m.dimension)) as info:
            builds = lib.scn_rulebook_build_count()
            check(lib.scn_md_submanifold_rulebook(m._h, sizes(inputSize), sizes(filterSize), _stream(), None))
            info["built"] = lib.scn_rulebook_build_count() > builds  # False: served from the cache
        with _timed("conv", dict(op="submanifold", n_in=n, n_out=n, cin=cin, cout=cout, groups=groups,
                                 offsets=w.size(0), precision=_precision)) as info:
            if epilogue is None:
                check(lib.scn_submanifold_convolution_forward(
                    m._h, sizes(inputSize), sizes(filterSize), _ptr(f), _ptr(output_features), _ptr(w), _ptr(b),
                    groups * cin, groups * cout, groups, _precision, _stream(), C.byref(macs)))
            else:
                sc, sh, leak = _epilogue_args(epilogue, f, groups * cout)
                info["fused_bn"] = True
                check(lib.scn_submanifold_convolution_bn_forward(
                    m._h, sizes(inputSize), sizes(filterSize), _ptr(f), _ptr(output_features), _ptr(w), _ptr(b),
                    sc, sh, leak, groups * cin, groups * cout, groups, _precision, _stream(), C.byref(macs)))
            result = _macs_result(m, macs)
            if Profile.active is not None:
                info["macs"] = float(result)
            info["kernel"] = _KERNEL_NAMES[lib.scn_last_conv_kernel()]
    return result


def strided_chain(m, inputSize, filterSize, filterStride, levels, device):
    """Not in the reference: a hint from a caller that knows its network goes `levels` levels down with
    the same downsampling (a U-Net's or ResNet's encoder).  The grids and rulebooks of those levels
    (Metadata<D>::getRuleBook, Metadata.cpp:492-518, once per level) are built in one enqueued chain with
    a single wait for all the level counts; the Convolutions then find theirs in the cache.  Returns the
    number of levels built (0 when there was nothing to chain)."""
    if levels < 2:
        return 0
    built = C.c_int(0)
    with _on_device(device), _timed("rules_strided", dict(
            sites=0, sites_out=0, offsets=int(torch.as_tensor(filterSize).prod()), dim=m.dimension)) as info:
        check(lib.scn_md_strided_chain(m._h, sizes(inputSize), sizes(filterSize), sizes(filterStride), int(levels),
                                       _stream(), C.byref(built)))
        info["built"] = built.value > 0
        info["levels"] = built.value
        # started earlier on the side stream: its kernels ran beside other operators' and are in their times
        info["overlapped"] = bool(getattr(m, "chain_started", False))
        if built.value and Profile.active is not None:  # all the levels' sites are this call's work
            cur = [int(v) for v in inputSize]
            for _ in range(built.value):
                nxt = [(c - int(fs)) // int(st) + 1 for c, fs, st in zip(cur, filterSize, filterStride)]
                info["sites"] += m.getNActive(torch.LongTensor(cur))
                info["sites_out"] += m.getNActive(torch.LongTensor(nxt))
                cur = nxt
    return built.value


def SubmanifoldConvolution_joined(inputSize, filterSize, m, inputs, output_features, weight, bias, prologue=None,
                                  epilogue=None):
    """SubmanifoldConvolution of the column-wise concatenation of two feature matrices over the same sites (a
    JoinTable in front of the layer), optionally through an eval-mode BatchNorm in between (`prologue`) and with the
    one behind in its store (`epilogue`): scn_submanifold_convolution_joined_forward.  Not in the reference.
    Returns None when the shapes are not ones the call takes (the caller then joins first)."""
    if len(inputs) != 2 or weight.size(1) != 1:
        return None
    fa, fb = (_features(f, "input_features") for f in inputs)
    ca, cb = fa.size(1), fb.size(1)
    if fa.size(0) != fb.size(0) or ca % 8 or cb % 4 or fa.device != fb.device or weight.size(2) != ca + cb:
        return None
    w = _features(weight.detach(), "weight")
    b = _optional(bias, fa, "bias")
    n, cout = fa.size(0), w.size(3)
    macs = C.c_double()
    with _on_device(fa.device):
        if n != m.getNActive(inputSize):
            raise RuntimeError("features have %d rows, metadata has %d active sites" % (n, m.getNActive(inputSize)))
        output_features.resize_(n, cout)
        psc, psh, pleak = _epilogue_args(prologue, fa, ca + cb) if prologue is not None else (None, None, 1.0)
        sc, sh, leak = _epilogue_args(epilogue, fa, cout) if epilogue is not None else (None, None, 1.0)
        with _timed("conv", dict(op="submanifold", n_in=n, n_out=n, cin=ca + cb, cout=cout, groups=1, offsets=w.size(0),
                                 precision=_precision, joined=True, fused_bn=epilogue is not None,
                                 fused_bn_in_front=prologue is not None)) as info:
            check(lib.scn_submanifold_convolution_joined_forward(
                m._h, sizes(inputSize), sizes(filterSize), _ptr(fa), ca, _ptr(fb), cb, _ptr(output_features), _ptr(w),
                _ptr(b), psc, psh, pleak, sc, sh, leak, cout, _precision, _stream(), C.byref(macs)))
            result = _macs_result(m, macs)
            if Profile.active is not None:
                info["macs"] = float(result)
                info["kernel"] = _KERNEL_NAMES[lib.scn_last_conv_kernel()]
    return result


def strided_chain_start(m, inputSize, filterSize, filterStride, levels, device):
    """strided_chain without the wait (scn_md_strided_chain_start): the chain's kernels go to the library's side
    stream behind what the current stream holds now and run beside what is enqueued next; the call that first
    needs one of the levels takes them over.  Not in the reference."""
    if levels < 2:
        return
    with _on_device(device):
        check(lib.scn_md_strided_chain_start(m._h, sizes(inputSize), sizes(filterSize), sizes(filterStride),
                                             int(levels), _stream()))
    m.chain_started = True


def Convolution_updateOutput(inputSize, outputSize, filterSize, filterStride, m, input_features,
                             output_features, weight, bias, epilogue=None, prologue=None):
    """sparseconvnet.h:87-92.  `epilogue` (not in the reference): see batchnorm_fold.  `prologue` (not in the
    reference): the same triple for an eval-mode BatchNorm in FRONT of the layer (scn_convolution_bn_bn_forward)."""
    f, w, b, groups, cin, cout = _conv_args(input_features, weight, bias)
    macs = C.c_double()
    n_out = C.c_int64()
    with _on_device(f.device):
        if f.size(0) != m.getNActive(inputSize):
            raise RuntimeError("features have %d rows, metadata has %d active sites"
                               % (f.size(0), m.getNActive(inputSize)))
        with _timed("rules_strided", dict(sites=f.size(0), offsets=w.size(0), dim=m.dimension)) as info:
            builds = lib.scn_rulebook_build_count()
            check(lib.scn_md_strided_rulebook(m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize),
                                              sizes(filterStride), _stream(), C.byref(n_out), None))
            info["sites_out"] = n_out.value
            info["built"] = lib.scn_rulebook_build_count() > builds
        output_features.resize_(n_out.value, groups * cout)
        with _timed("conv", dict(op="strided", n_in=f.size(0), n_out=n_out.value, cin=cin, cout=cout,
                                 groups=groups, offsets=w.size(0), precision=_precision)) as info:
            if prologue is not None:
                psc, psh, pleak = _epilogue_args(prologue, f, groups * cin)
                sc, sh, leak = _epilogue_args(epilogue, f, groups * cout) if epilogue is not None else (None, None, 1.0)
                info["fused_bn_in_front"] = True
                info["fused_bn"] = epilogue is not None
                check(lib.scn_convolution_bn_bn_forward(
                    m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
                    _ptr(output_features), _ptr(w), _ptr(b), psc, psh, pleak, sc, sh, leak, groups * cin,
                    groups * cout, groups, _precision, _stream(), C.byref(macs)))
            elif epilogue is None:
                check(lib.scn_convolution_forward(
                    m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
                    _ptr(output_features), _ptr(w), _ptr(b), groups * cin, groups * cout, groups, _precision,
                    _stream(), C.byref(macs)))
            else:
                sc, sh, leak = _epilogue_args(epilogue, f, groups * cout)
                info["fused_bn"] = True
                check(lib.scn_convolution_bn_forward(
                    m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
                    _ptr(output_features), _ptr(w), _ptr(b), sc, sh, leak, groups * cin, groups * cout, groups,
                    _precision, _stream(), C.byref(macs)))
            result = _macs_result(m, macs)
            if Profile.active is not None:
                info["macs"] = float(result)
            info["kernel"] = _KERNEL_NAMES[lib.scn_last_conv_kernel()]
    return result


def Deconvolution_updateOutput(inputSize, outputSize, filterSize, filterStride, m, input_features,
                               output_features, weight, bias, epilogue=None):
    """sparseconvnet.h:149-154.  `epilogue` (not in the reference): see batchnorm_fold."""
    f, w, b, groups, cin, cout = _conv_args(input_features, weight, bias)
    macs = C.c_double()
    with _on_device(f.device):
        # same rulebook as the Convolution that made `inputSize` out of `outputSize`
        check(lib.scn_md_strided_rulebook(m._h, sizes(outputSize), sizes(inputSize), sizes(filterSize),
                                          sizes(filterStride), _stream(), None, None))
        if f.size(0) != m.getNActive(inputSize):
            raise RuntimeError("features have %d rows, metadata has %d active sites"
                               % (f.size(0), m.getNActive(inputSize)))
        n_fine = m.getNActive(outputSize)
        output_features.resize_(n_fine, groups * cout)
        with _timed("conv", dict(op="deconvolution", n_in=f.size(0), n_out=n_fine, cin=cin, cout=cout,
                                 groups=groups, offsets=w.size(0), precision=_precision)) as info:
            if epilogue is None:
                check(lib.scn_deconvolution_forward(
                    m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
                    _ptr(output_features), _ptr(w), _ptr(b), groups * cin, groups * cout, groups, _precision,
                    _stream(), C.byref(macs)))
            else:
                sc, sh, leak = _epilogue_args(epilogue, f, groups * cout)
                info["fused_bn"] = True
                check(lib.scn_deconvolution_bn_forward(
                    m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
                    _ptr(output_features), _ptr(w), _ptr(b), sc, sh, leak, groups * cin, groups * cout, groups,
                    _precision, _stream(), C.byref(macs)))
            result = _macs_result(m, macs)
            if Profile.active is not None:
                info["macs"] = float(result)
            info["kernel"] = _KERNEL_NAMES[lib.scn_last_conv_kernel()]
    return result


def BatchNormalization_updateOutput(input_features, output_features, saveMean, saveInvStd, runningMean,
                                    runningVar, weight, bias, eps, momentum, train, leakiness):
    """sparseconvnet.h:22-26.  Accepts a column slice of a wider matrix (row stride > planes),
    as the reference does (CPU/BatchNormalization.cpp:9-10)."""
    f = input_features
    if not f.is_cuda or f.dtype != torch.float32 or f.dim() != 2 or (f.numel() and f.stride(1) != 1):
        raise RuntimeError("input_features must be a CUDA float32 matrix with unit column stride")
    n, c = f.size(0), f.size(1)
    with _on_device(f.device):
        output_features.resize_(n, c)
        saveMean.resize_(c)
        saveInvStd.resize_(c)
        if n == 0:
            return
        w = _optional(weight, f, "weight")
        b = _optional(bias, f, "bias")
        with _timed("batchnorm", dict(rows=n, planes=c)):
            check(lib.scn_batchnorm_forward(
                _ptr(f), _ptr(output_features), n, c, f.stride(0), output_features.stride(0), _ptr(saveMean),
                _ptr(saveInvStd), _ptr(_features(runningMean, "runningMean")),
                _ptr(_features(runningVar, "runningVar")), _ptr(w), _ptr(b), float(eps), float(momentum),
                int(bool(train)), float(leakiness), _stream()))


def batchnorm_concat(inputs, running_mean, running_var, weight, bias, eps, leakiness):
    """Eval-mode BatchNormalization of the column-wise concatenation of two matrices (a JoinTable followed
    by a BatchNorm) without materialising the concatenation: same arithmetic as
    BatchNormalization_updateOutput on torch.cat(inputs, 1) (CPU/BatchNormalization.cpp:41-61), one read
    and one write of the activation instead of two each.  Not in the reference.  Returns None when the
    shapes are not ones the fused kernel takes (the caller then joins and normalises in two steps)."""
    if len(inputs) != 2:
        return None
    fa, fb = (_features(f, "input_features") for f in inputs)
    if fa.size(0) != fb.size(0) or fa.size(1) % 4 or fb.size(1) % 4 or fa.device != fb.device:
        return None
    n, ca, cb = fa.size(0), fa.size(1), fb.size(1)
    out = fa.new_empty(n, ca + cb)
    w = _optional(weight, fa, "weight")
    b = _optional(bias, fa, "bias")
    with _on_device(fa.device):
        with _timed("batchnorm", dict(rows=n, planes=ca + cb, joined=True)):
            check(lib.scn_batchnorm_join_forward(_ptr(fa), ca, _ptr(fb), cb, _ptr(out), n,
                                                 _ptr(_features(running_mean, "runningMean")),
                                                 _ptr(_features(running_var, "runningVar")), _ptr(w), _ptr(b),
                                                 float(eps), float(leakiness), _stream()))
    return out


def _conv_backward_args(input_features, d_input_features, d_output_features, weight, d_weight, d_bias):
    f, w, _, groups, cin, cout = _conv_args(input_features, weight, torch.empty(0))
    go = _features(d_output_features, "d_output_features")
    dw = _features(d_weight, "d_weight")
    if dw.shape != w.shape:
        raise RuntimeError("d_weight must have the shape of weight")
    db = _features(d_bias, "d_bias") if d_bias is not None and d_bias.numel() else None
    d_input_features.resize_(f.size(0), groups * cin)
    return f, w, go, dw, db, groups, cin, cout


def SubmanifoldConvolution_backward(inputSize, filterSize, m, input_features, d_input_features,
                                    d_output_features, weight, d_weight, d_bias):
    """sparseconvnet.h:106-114.  fp32; gradients are overwritten."""
    f, w, go, dw, db, groups, cin, cout = _conv_backward_args(input_features, d_input_features,
                                                             d_output_features, weight, d_weight, d_bias)
    with _on_device(f.device):
        check(lib.scn_submanifold_convolution_backward(
            m._h, sizes(inputSize), sizes(filterSize), _ptr(f), _ptr(d_input_features), _ptr(go), _ptr(w),
            _ptr(dw), _ptr(db), groups * cin, groups * cout, groups, _stream()))


def Convolution_backward(inputSize, outputSize, filterSize, filterStride, m, input_features, d_input_features,
                         d_output_features, weight, d_weight, d_bias):
    """sparseconvnet.h:94-104."""
    f, w, go, dw, db, groups, cin, cout = _conv_backward_args(input_features, d_input_features,
                                                             d_output_features, weight, d_weight, d_bias)
    with _on_device(f.device):
        check(lib.scn_convolution_backward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
            _ptr(d_input_features), _ptr(go), _ptr(w), _ptr(dw), _ptr(db), groups * cin, groups * cout, groups,
            _stream()))


def Deconvolution_backward(inputSize, outputSize, filterSize, filterStride, m, input_features, d_input_features,
                           d_output_features, weight, d_weight, d_bias):
    """sparseconvnet.h:156-166."""
    f, w, go, dw, db, groups, cin, cout = _conv_backward_args(input_features, d_input_features,
                                                             d_output_features, weight, d_weight, d_bias)
    with _on_device(f.device):
        check(lib.scn_deconvolution_backward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(filterSize), sizes(filterStride), _ptr(f),
            _ptr(d_input_features), _ptr(go), _ptr(w), _ptr(dw), _ptr(db), groups * cin, groups * cout, groups,
            _stream()))


def MaxPooling_updateOutput(inputSize, outputSize, poolSize, poolStride, m, input_features,
                            output_features, nFeaturesToDrop):
    """sparseconvnet.h:198-201."""
    f = _features(input_features, "input_features")
    n_out = C.c_int64()
    with _on_device(f.device):
        check(lib.scn_md_strided_rulebook(m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize),
                                          sizes(poolStride), _stream(), C.byref(n_out), None))
        output_features.resize_(n_out.value, f.size(1) - int(nFeaturesToDrop))
        check(lib.scn_max_pooling_forward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(f),
            _ptr(output_features), f.size(1), int(nFeaturesToDrop), _stream()))


def AveragePooling_updateOutput(inputSize, outputSize, poolSize, poolStride, m, input_features,
                                output_features, nFeaturesToDrop):
    """sparseconvnet.h (AveragePooling_updateOutput), CPU/AveragePooling.cpp:38-61."""
    f = _features(input_features, "input_features")
    n_out = C.c_int64()
    with _on_device(f.device):
        check(lib.scn_md_strided_rulebook(m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize),
                                          sizes(poolStride), _stream(), C.byref(n_out), None))
        output_features.resize_(n_out.value, f.size(1) - int(nFeaturesToDrop))
        check(lib.scn_average_pooling_forward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(f),
            _ptr(output_features), f.size(1), int(nFeaturesToDrop), _stream()))


def UnPooling_updateOutput(inputSize, outputSize, poolSize, poolStride, m, input_features, output_features,
                           nFeaturesToDrop):
    """sparseconvnet.h (UnPooling_updateOutput), CPU/UnPooling.cpp:35-59: inputSize is the coarse scale,
    outputSize the fine one (its grid must exist already)."""
    f = _features(input_features, "input_features")
    with _on_device(f.device):
        output_features.resize_(m.getNActive(outputSize), f.size(1) - int(nFeaturesToDrop))
        check(lib.scn_unpooling_forward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(f),
            _ptr(output_features), f.size(1), int(nFeaturesToDrop), _stream()))


def SparseToDense_updateOutput(inputSize, m, input_features, output_features, nPlanes):
    """sparseconvnet.h:220-222.  Output [batch, nPlanes, *inputSize]."""
    f = _features(input_features, "input_features")
    with _on_device(f.device):
        shape = [m.getBatchSize(inputSize), int(nPlanes)] + [int(v) for v in inputSize]
        output_features.resize_(*shape)
        if f.dim() == 2:
            if f.size(1) != nPlanes:
                raise RuntimeError("features have %d planes, nPlanes is %d" % (f.size(1), nPlanes))
            check(lib.scn_sparse_to_dense_forward(m._h, sizes(inputSize), _ptr(f), _ptr(output_features),
                                                  int(nPlanes), _stream()))
        else:
            output_features.zero_()


def rows_affine_supported(features, weight):
    """True when scn_rows_affine_forward takes the product features @ weight (fp32 on a GPU, at most 32
    output planes, input planes a multiple of four up to 256)."""
    return (features.is_cuda and features.dtype == torch.float32 and weight.dtype == torch.float32
            and weight.dim() == 2 and features.dim() == 2 and features.size(1) == weight.size(0)
            and 1 <= weight.size(1) <= 32 and weight.size(0) % 4 == 0 and 4 <= weight.size(0) <= 256)


def rows_affine(features, weight, bias=None, out=None):
    """out = bias + features @ weight for a weight matrix [nIn, nOut] with nOut <= 32, in one pass over
    the rows (a NetworkInNetwork with few output planes, CPU/NetworkInNetwork.cpp:7-23; the per-voxel
    class head of a segmentation network, with torch.nn.Linear's weight transposed).  Forward only.
    ``out`` may be any [n, nOut] fp32 matrix with contiguous rows, for instance a block of a larger buffer."""
    f = _features(features, "features")
    w = _features(weight, "weight")
    if not rows_affine_supported(f, w):
        raise RuntimeError("rows_affine: unsupported shapes %s x %s" % (tuple(f.shape), tuple(w.shape)))
    n, cout = f.size(0), w.size(1)
    if out is None:
        out = f.new_empty(n, cout)
    elif out.shape != (n, cout) or not out.is_contiguous() or out.dtype != torch.float32 or out.device != f.device:
        raise RuntimeError("rows_affine: out must be a contiguous fp32 [%d, %d] matrix on %s" % (n, cout, f.device))
    b = _features(bias, "bias") if bias is not None else None
    if b is not None and b.numel() != cout:
        raise RuntimeError("rows_affine: bias must have %d entries" % cout)
    with _on_device(f.device):
        with _timed("rows_affine", dict(rows=n, nin=f.size(1), nout=cout)):
            check(lib.scn_rows_affine_forward(_ptr(f), _ptr(out), n, f.size(1), cout, _ptr(w), _ptr(b), _stream()))
    return out


def NetworkInNetwork_updateOutput(input_features, output_features, weight, bias):
    """sparseconvnet.h:51-53.  The reference itself hands this 1x1 convolution to the dense
    matrix library (CPU/NetworkInNetwork.cpp:7-23: ``addmm_``); so does this."""
    f = _features(input_features, "input_features")
    n, cout = f.size(0), weight.size(1)
    output_features.resize_(n, cout)
    if rows_affine_supported(f, weight):
        rows_affine(f, weight.detach(), bias.detach() if bias is not None and bias.numel() else None,
                    out=output_features)
        return float(n * f.size(1) * cout)
    if bias is not None and bias.numel():
        output_features.copy_(bias.detach().expand(n, cout))
    else:
        output_features.zero_()
    if n:
        output_features.addmm_(f, weight.detach())
    return float(n * f.size(1) * cout)


def BatchNormalization_backward(input_features, d_input_features, output_features, d_output_features, saveMean,
                                saveInvStd, runningMean, runningVar, weight, bias, d_weight, d_bias, leakiness):
    """sparseconvnet.h:28-38.  d_output_features is left untouched (the reference scales it in place)."""
    f = input_features
    n, c = f.size(0), f.size(1)
    d_input_features.resize_(n, c)
    w = _optional(weight, f, "weight")
    with _on_device(f.device):
        check(lib.scn_batchnorm_backward(
            _ptr(f), _ptr(d_input_features), _ptr(output_features), _ptr(d_output_features), n, c,
            f.stride(0) if n else c, output_features.stride(0) if n else c, _ptr(saveMean), _ptr(saveInvStd),
            _ptr(w), _ptr(d_weight), _ptr(d_bias), float(leakiness), _stream()))


def _sum_over_ranks(t, group):
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


def BatchNormalization_updateOutput_acrossRanks(input_features, output_features, saveMean, saveInvStd, runningMean,
                                                runningVar, weight, bias, eps, momentum, leakiness, group=None,
                                                reduce=_sum_over_ranks):
    """Training-mode BatchNormalization_updateOutput (CPU/BatchNormalization.cpp:12-62) whose statistics cover the
    rows of every rank of `group`: each rank sums its rows, one all-reduce of 2 x planes + 1 doubles adds the sums
    and the row counts, every rank normalises its own rows with the shared mean and variance and makes the same
    update of the running statistics.  Not in the reference (single device).  A rank without rows takes part in
    the all-reduce.  `reduce(tensor, group)` adds a tensor over the ranks in place.  The host never reads the
    total row count: it stays on the device, behind the sums.  Returns the summed array (the backward call
    wants it for the count)."""
    f = input_features
    if not f.is_cuda or f.dtype != torch.float32 or f.dim() != 2 or (f.numel() and f.stride(1) != 1):
        raise RuntimeError("input_features must be a CUDA float32 matrix with unit column stride")
    n, c = f.size(0), f.size(1)
    with _on_device(f.device):
        output_features.resize_(n, c)
        saveMean.resize_(c)
        saveInvStd.resize_(c)
        sums = torch.empty(2 * c + 1, dtype=torch.float64, device=f.device)
        sums[2 * c] = n
        check(lib.scn_batchnorm_moments(_ptr(f), n, c, f.stride(0) if n else c, _ptr(sums), _stream()))
        reduce(sums, group)
        w = _optional(weight, f, "weight")
        b = _optional(bias, f, "bias")
        check(lib.scn_batchnorm_forward_moments(
            _ptr(f), _ptr(output_features), n, -1, c, f.stride(0) if n else c,
            output_features.stride(0) if n else c, _ptr(sums), _ptr(saveMean), _ptr(saveInvStd),
            _ptr(_features(runningMean, "runningMean")), _ptr(_features(runningVar, "runningVar")), _ptr(w), _ptr(b),
            float(eps), float(momentum), float(leakiness), _stream()))
    return sums


def BatchNormalization_backward_acrossRanks(input_features, d_input_features, output_features, d_output_features,
                                            saveMean, saveInvStd, weight, d_weight, d_bias, leakiness, forward_sums,
                                            group=None, reduce=_sum_over_ranks):
    """Backward of BatchNormalization_updateOutput_acrossRanks (the formula of CPU/BatchNormalization.cpp:64-107
    with the two sums taken over all ranks).  d_weight / d_bias receive THIS rank's share, so that summing the
    parameter gradients over the ranks, as for every other parameter, gives the gradient of the whole batch.
    `forward_sums`: what the forward call returned."""
    f = input_features
    n, c = f.size(0), f.size(1)
    d_input_features.resize_(n, c)
    w = _optional(weight, f, "weight")
    with _on_device(f.device):
        local = torch.empty(2 * c + 1, dtype=torch.float64, device=f.device)
        check(lib.scn_batchnorm_backward_sums(
            _ptr(f), _ptr(output_features), _ptr(d_output_features), n, c, f.stride(0) if n else c,
            output_features.stride(0) if n else c, _ptr(saveMean), float(leakiness), _ptr(local), _stream()))
        local[2 * c] = 0
        total = local.clone()
        reduce(total, group)
        total[2 * c] = forward_sums[2 * c]
        check(lib.scn_batchnorm_backward_sums_apply(
            _ptr(f), _ptr(d_input_features), _ptr(output_features), _ptr(d_output_features), n, -1, c,
            f.stride(0) if n else c, output_features.stride(0) if n else c, _ptr(saveMean), _ptr(saveInvStd),
            _ptr(w), _ptr(local), _ptr(total), _ptr(d_weight), _ptr(d_bias), float(leakiness), _stream()))


def InputLayer_updateGradInput(m, d_input_features, d_output_features):
    """CPU/IOLayers.cpp:74-93 (and BLInputLayer_updateGradInput, :165-186, reshaped by the caller)."""
    go = _features(d_output_features, "d_output_features")
    d_input_features.resize_(m.n_input_rows, go.size(1))
    with _on_device(go.device):
        check(lib.scn_input_layer_backward(m._h, _ptr(d_input_features), m.n_input_rows, _ptr(go), go.size(0),
                                           go.size(1), _stream()))


def OutputLayer_updateGradInput(m, d_input_features, d_output_features):
    """CPU/IOLayers.cpp:116-136 (and BLOutputLayer_updateGradInput): d_output [points..., planes];
    d_input_features must already have its [n_active, planes] shape."""
    go = _features(d_output_features, "d_output_features")
    with _on_device(go.device):
        check(lib.scn_output_layer_backward(m._h, _ptr(d_input_features), d_input_features.size(0), _ptr(go),
                                            m.n_input_rows, go.size(-1), _stream()))


def MaxPooling_updateGradInput(inputSize, outputSize, poolSize, poolStride, m, input_features, d_input_features,
                               output_features, d_output_features, nFeaturesToDrop):
    """sparseconvnet.h:203-212."""
    f = _features(input_features, "input_features")
    d_input_features.resize_(f.size(0), f.size(1))
    with _on_device(f.device):
        check(lib.scn_max_pooling_backward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(f),
            _ptr(d_input_features), _ptr(_features(output_features, "output_features")),
            _ptr(_features(d_output_features, "d_output_features")), f.size(1), int(nFeaturesToDrop), _stream()))


def AveragePooling_updateGradInput(inputSize, outputSize, poolSize, poolStride, m, input_features,
                                   d_input_features, d_output_features, nFeaturesToDrop):
    """sparseconvnet.h:81-92."""
    f = _features(input_features, "input_features")
    d_input_features.resize_(f.size(0), f.size(1))
    with _on_device(f.device):
        check(lib.scn_average_pooling_backward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(d_input_features),
            _ptr(_features(d_output_features, "d_output_features")), f.size(1), int(nFeaturesToDrop), _stream()))


def UnPooling_updateGradInput(inputSize, outputSize, poolSize, poolStride, m, d_input_features, d_output_features,
                              nFeaturesToDrop):
    """sparseconvnet.h:235-242: d_input_features must already have the input's shape."""
    go = _features(d_output_features, "d_output_features")
    with _on_device(go.device):
        check(lib.scn_unpooling_backward(
            m._h, sizes(inputSize), sizes(outputSize), sizes(poolSize), sizes(poolStride), _ptr(d_input_features),
            _ptr(go), d_input_features.size(1), int(nFeaturesToDrop), _stream()))


def SparseToDense_updateGradInput(inputSize, m, input_features, d_input_features, d_output_features):
    """sparseconvnet.h:224-228."""
    go = _features(d_output_features, "d_output_features")
    d_input_features.resize_(input_features.size(0), input_features.size(1))
    with _on_device(go.device):
        check(lib.scn_sparse_to_dense_backward(m._h, sizes(inputSize), _ptr(d_input_features), _ptr(go),
                                               input_features.size(1), _stream()))


def _training_only(*a, **k):
    raise NotImplementedError("this backward pass is not part of sparseconvnet_b200 yet")


NetworkInNetwork_updateGradInput = NetworkInNetwork_accGradParameters = _training_only  # torch autograd does these
