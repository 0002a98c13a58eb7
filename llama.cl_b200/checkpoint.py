"""Reader / writer of the reference's saved models.

The reference saves a model with ``pickle.dump(self.__dict__, f)`` (``chatllama/main.py:305-308``).  What is
inside: its op objects (``llmop_fc_q4a`` & co., ``chatllama/main.py:158-238``, pickled under ``__main__``
because the reference runs as a script, or under ``main`` when it was imported) whose attributes are
``llmops.tensor`` objects; a tensor pickles as ``(numpy array,)`` (``ops/main.cpp:129-136``).

``load`` reads such a file without the reference installed: every ``llmops.tensor`` becomes a ``HostTensor``
(a numpy array holder) and every op object a plain attribute holder that remembers its class name.  The packed
FC weights in it are the reference's bytes, which are this library's bytes too, so ``fc_ops`` hands them to the
GPU as they are -- no repacking -- and returns runnable ``ops.llmop_fc_q4a`` objects.  ``save`` writes the
object graph back; a file that was loaded and saved unchanged is byte-identical to the original (same pickle
protocol, same class names, same order), so the reference can load what this library wrote.

Everything here is host-side format work; nothing touches the GPU until ``fc_ops`` is called.
"""
from __future__ import annotations

import io
import pickle
import sys
import types

import numpy as np

_TENSOR_MODULE, _TENSOR_NAME = "llmops", "tensor"
_OP_MODULES = ("__main__", "main")  # where the reference's op classes are found in a pickle


def _canonical(array) -> np.ndarray:
    """Contiguous, and carrying numpy's own dtype object for its type.  A dtype that comes out of a pickle is a
    separate object; the pickler shares objects by identity, so a model in which loaded and freshly made arrays
    mix would otherwise be written with the dtype spelled out more than once -- not as the reference writes it."""
    a = np.ascontiguousarray(array)
    return a.view(np.dtype(a.dtype.str))


class HostTensor:
    """Stand-in for ``llmops.tensor`` on the host: holds the numpy array the reference pickled."""

    __slots__ = ("array",)

    def __init__(self, array) -> None:
        self.array = _canonical(array)

    # the pickle protocol of ops/main.cpp:129-136: state = (numpy array,)
    def __getstate__(self):
        return (self.array,)

    def __setstate__(self, state) -> None:
        self.array = _canonical(state[0])

    @property
    def shape(self):
        return list(self.array.shape)

    @property
    def item_size(self) -> int:
        return self.array.dtype.itemsize

    def numel(self) -> int:
        return int(self.array.size)

    def numpy(self) -> np.ndarray:
        return self.array

    def __repr__(self) -> str:
        return f"HostTensor(shape={self.shape}, dtype={self.array.dtype})"


# for the pickler this class IS llmops.tensor
HostTensor.__module__ = _TENSOR_MODULE
HostTensor.__qualname__ = HostTensor.__name__ = _TENSOR_NAME


class _OpBase:
    """Attribute holder for a pickled op object of the reference; one subclass per (module, class name)."""

    def __repr__(self) -> str:
        return f"<{type(self).__module__}.{type(self).__name__} {sorted(self.__dict__)}>"


_op_classes: dict[tuple[str, str], type] = {}


def _op_class(module: str, name: str) -> type:
    key = (module, name)
    if key not in _op_classes:
        cls = type(name, (_OpBase,), {})
        cls.__module__, cls.__qualname__ = module, name
        _op_classes[key] = cls
    return _op_classes[key]


# Everything else a saved model refers to: numpy's array reconstruction.  No other global is resolved, so that a
# file from an unknown source cannot name a callable of its choosing (the reference's own pickle.load can).
_NUMPY_GLOBALS = {(m, n) for m in ("numpy", "numpy.core.multiarray", "numpy._core.multiarray", "numpy.core.numeric",
                                   "numpy._core.numeric")
                  for n in ("_reconstruct", "ndarray", "dtype", "scalar", "_frombuffer")}


class _Unpickler(pickle.Unpickler):
    def find_class(self, module: str, name: str):
        if module == _TENSOR_MODULE and name == _TENSOR_NAME:
            return HostTensor
        if module in _OP_MODULES and name.startswith("llmop_"):
            return _op_class(module, name)
        if (module, name) in _NUMPY_GLOBALS:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"a saved model does not refer to {module}.{name}: refusing to resolve it")


def load(path_or_file):
    """The object graph of a saved model (normally the dict of ``Model.__dict__``)."""
    if hasattr(path_or_file, "read"):
        return _Unpickler(path_or_file).load()
    with open(path_or_file, "rb") as f:
        return _Unpickler(f).load()


def loads(data: bytes):
    return _Unpickler(io.BytesIO(data)).load()


class _borrowed_modules:
    """While pickling, the class names of the stand-ins must resolve to the stand-ins: ``llmops.tensor`` and
    the op classes under the module they were loaded from.  Existing modules of those names get the
    attributes for the duration and are restored afterwards."""

    def __init__(self) -> None:
        self._undo: list = []

    def _set(self, module: str, name: str, value) -> None:
        mod = sys.modules.get(module)
        if mod is None:
            mod = types.ModuleType(module)
            sys.modules[module] = mod
            self._undo.append(("module", module, None))
        had = hasattr(mod, name)
        self._undo.append(("attr", mod, (name, getattr(mod, name, None), had)))
        setattr(mod, name, value)

    def __enter__(self):
        self._set(_TENSOR_MODULE, _TENSOR_NAME, HostTensor)
        for (module, name), cls in list(_op_classes.items()):
            self._set(module, name, cls)
        return self

    def __exit__(self, *exc) -> None:
        for kind, a, b in reversed(self._undo):
            if kind == "attr":
                name, old, had = b
                if had:
                    setattr(a, name, old)
                else:
                    delattr(a, name)
            else:
                sys.modules.pop(a, None)


def dumps(obj, protocol: int = 4) -> bytes:
    """Pickle bytes as the reference would write them (its ``pickle.dump`` default, protocol 4)."""
    with _borrowed_modules():
        return pickle.dumps(obj, protocol=protocol)


def save(obj, path: str, protocol: int = 4) -> None:
    data = dumps(obj, protocol)
    with open(path, "wb") as f:
        f.write(data)


def new_op(name: str, module: str = "__main__", **attrs):
    """A fresh op object of the reference's class ``name`` (for writing models the reference can load)."""
    op = _op_class(module, name)()
    op.__dict__.update(attrs)
    return op


# ---------------------------------------------------------------------------------------------------------
def walk_ops(obj, prefix: str = ""):
    """Yields ``(dotted path, op object)`` for every reference op in dicts / lists of a loaded model."""
    if isinstance(obj, _OpBase):
        yield prefix, obj
    elif isinstance(obj, dict):
        for k, v in obj.items():
            yield from walk_ops(v, f"{prefix}.{k}" if prefix else str(k))
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            yield from walk_ops(v, f"{prefix}.{i}" if prefix else str(i))


def fc_ops(model, device="cuda") -> dict:
    """``{path: ops.llmop_fc_q4a}`` for every ``llmop_fc_q4a`` of a loaded model, packed weights copied to
    ``device`` byte for byte (the block type is recovered from the block size)."""
    import torch

    from . import _cabi
    from .ops import llmop_fc_q4a

    out = {}
    for path, op in walk_ops(model):
        if type(op).__name__ != "llmop_fc_q4a":
            continue
        packed = op.weight.numpy()
        if packed.dtype != np.int8 or packed.ndim != 3:
            raise RuntimeError(f"{path}: packed weight is {packed.dtype}{list(packed.shape)}, expected int8 [Ng, Kg, BS]")
        _cabi.infer_variant(packed.shape[2])  # raises on an unknown block size
        gpu = llmop_fc_q4a.__new__(llmop_fc_q4a)
        gpu.weight = torch.from_numpy(np.ascontiguousarray(packed)).to(device)
        bias = getattr(op, "bias", None)
        gpu.bias = None
        if isinstance(bias, HostTensor) and bias.numel() > 0:
            gpu.bias = torch.from_numpy(np.ascontiguousarray(bias.numpy(), dtype=np.float32)).to(device)
        gpu.N = int(op.N)
        out[path] = gpu
    return out


def embedding_ops(model, device="cuda") -> dict:
    """``{path: ops.llmop_embedding_q8c}`` for every ``llmop_embedding_q8c`` of a loaded model: its int8 codes and
    fp32 scales copied to ``device`` as they are."""
    import torch

    from .ops import llmop_embedding_q8c

    out = {}
    for path, op in walk_ops(model):
        if type(op).__name__ != "llmop_embedding_q8c":
            continue
        codes, scales = op.weight.numpy(), op.scales.numpy()
        if codes.dtype != np.int8 or codes.ndim != 2 or scales.dtype != np.float32 or scales.shape != codes.shape[:1]:
            raise RuntimeError(f"{path}: expected int8 [V, E] codes and fp32 [V] scales, got "
                               f"{codes.dtype}{list(codes.shape)} / {scales.dtype}{list(scales.shape)}")
        gpu = llmop_embedding_q8c.__new__(llmop_embedding_q8c)
        gpu.weight = torch.from_numpy(np.ascontiguousarray(codes)).to(device)
        gpu.scales = torch.from_numpy(np.ascontiguousarray(scales)).to(device)
        out[path] = gpu
    return out


def store_fc(op, gpu_op) -> None:
    """Writes a GPU op's packed weight (and bias, N) back into a loaded op object, e.g. after repacking."""
    op.weight = HostTensor(gpu_op.weight.detach().cpu().numpy())
    op.N = int(gpu_op.N)
    if gpu_op.bias is not None:
        op.bias = HostTensor(gpu_op.bias.detach().cpu().numpy())
