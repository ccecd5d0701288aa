"""Operator registration surface, API-compatible with ``iree.turbine.runtime.op_reg``.

The reference defines custom ops by subclassing ``CustomOp`` (signature / select / generate /
eager_execute) and decorating with ``CustomOp.register``
(iree/turbine/runtime/op_reg/base.py:97-252); registration defines the schema in a
``torch.library.Library``, installs a Meta implementation derived from ``select`` and a
per-dispatch-key trampoline (base.py:1041-1074), and records the op in ``ALL_CUSTOM_OP_REGS``.

That module cannot be imported without the IREE compiler, and everything below its trampoline
is an IREE JIT.  This module keeps the same class and method names and the same registration
semantics, but the trampoline ends in ``eager_execute`` -- the hook the reference itself uses for
ops implemented outside IREE (base.py:221-232, 1061-1064; precedent
iree/turbine/kernel/boo/ops/conv.py:35-86) -- and an op that does not implement it is an error
rather than a request to compile something.

Differences, all deliberate:
  * default dispatch keys are ``["CUDA"]`` only: there is no CPU implementation of these ops;
  * ``generate`` is optional (nothing emits IR here); AOT expansion is unsupported;
  * ``attr_bool`` exists (the reference accepts schema ``bool`` only through ``attr_int``
    because ``bool`` is an ``int`` in Python, base.py:540-548; both work here).
"""

from __future__ import annotations

import functools
import re
import threading
from abc import ABC, abstractmethod
from typing import Any, Callable, Optional, Sequence, Type, Union

import torch
from torch import Tensor

__all__ = [
    "ALL_CUSTOM_OP_REGS",
    "AttrArg",
    "CustomOp",
    "EagerKernelSelection",
    "EmptyOptionalTensorArg",
    "IntArg",
    "KernelSelection",
    "TensorArg",
    "TensorListArg",
    "def_library",
    "default_dispatch_keys",
]

_CONFIG_LOCK = threading.Lock()
_DEFINED: set[tuple[str, str]] = set()
_UNIQUE_COUNTERS: dict[tuple[str, str], int] = {}

# Fully qualified op name ("ns.name") -> CustomOp instance.
ALL_CUSTOM_OP_REGS: dict[str, "CustomOp"] = {}


def def_library(ns: str) -> torch.library.Library:
    """Creates a 'DEF' library that custom ops can be registered into (base.py:66-73)."""
    return torch.library.Library(ns, "DEF")


def default_dispatch_keys() -> list[str]:
    return ["CUDA"]


# ---------------------------------------------------------------------------------------------
# argument descriptors
# ---------------------------------------------------------------------------------------------
class TensorArg:
    """A tensor argument or result; ``spec_dims[i]`` is an int where dim i is specialised."""

    ir_arity = 1
    is_list = False

    def __init__(self, t: Tensor):
        self.t = t
        self.spec_dims: list[Optional[int]] = [None] * t.dim()
        self.maybe_tensor_value = t

    def specialize_all_dims(self):
        self.spec_dims = list(self.t.shape)

    def specialize_dims(self, *indices: int):
        for i in indices:
            self.spec_dims[i] = self.t.size(i)

    def generate_meta(self) -> Tensor:
        t = self.t
        return t.clone() if t.device.type == "meta" else torch.empty_like(t, device="meta")

    @property
    def spec_key(self) -> str:
        dims = ",".join("?" if d is None else str(d) for d in self.spec_dims)
        return f"tensor[{dims}:{self.t.dtype}]"

    def __repr__(self):
        return f"TensorArg(shape={list(self.t.shape)}, dtype={self.t.dtype}, spec_dims={self.spec_dims})"


class TensorListArg:
    ir_arity = 1
    is_list = True
    maybe_tensor_value = None

    def __init__(self, ts: list[Tensor]):
        self.ts = ts
        self.spec_dims = [[None] * t.dim() for t in ts]

    def generate_meta(self) -> list[Tensor]:
        return [torch.empty_like(t, device="meta") for t in self.ts]

    @property
    def spec_key(self) -> str:
        return "tensorlist[" + ";".join(f"{len(d)}:{t.dtype}" for d, t in zip(self.spec_dims, self.ts)) + "]"


class EmptyOptionalTensorArg:
    """Sentinel for an optional tensor that was not provided."""

    ir_arity = 0
    is_list = False
    maybe_tensor_value = None
    spec_key = "none"

    def generate_meta(self):
        return None

    def __repr__(self):
        return "EmptyOptionalTensorArg()"


class IntArg:
    ir_arity = 1
    is_list = False
    maybe_tensor_value = None

    def __init__(self, v: int):
        self.v = v
        self.spec_value: Optional[int] = None

    def generate_meta(self) -> int:
        return self.v

    @property
    def spec_key(self) -> str:
        return f"int<{self.spec_value}>"

    def __repr__(self):
        return f"IntArg({self.v}, spec_value={self.spec_value})"


class AttrArg:
    """A compile-time attribute; every distinct value is its own specialisation."""

    ir_arity = 0
    is_list = False
    maybe_tensor_value = None

    def __init__(self, v: object):
        self.v = v
        self.spec_value = v

    def generate_meta(self) -> object:
        return self.v

    @property
    def spec_key(self) -> str:
        return f"attr<{self.spec_value}>"

    def __repr__(self):
        return f"AttrArg(<{self.spec_value}>)"


# ---------------------------------------------------------------------------------------------
# kernel selection
# ---------------------------------------------------------------------------------------------
class KernelSelection(ABC):
    """Typed view of one call's arguments plus the declared results (base.py:255-468)."""

    def __init__(self, op: "CustomOp", arg_arity: int):
        self.op = op
        self.arg_descs: list = [None] * arg_arity
        self.inplace_tied_arg_descs: list = []
        self.result_descs: list = []
        self.variant = "default"

    def generate_meta_returns(self) -> Any:
        results = [d.generate_meta() for d in self.result_descs]
        if len(results) == 1:
            return results[0]
        return tuple(results) if results else None

    @property
    def spec_key(self) -> str:
        args = ",".join(d.spec_key if d is not None else "None" for d in self.arg_descs)
        rets = ",".join(d.spec_key if d is not None else "None" for d in self.result_descs)
        return f"{self.op.cache_key_base}::{self.variant}({args})->({rets})"

    def __repr__(self):
        return f"KernelSelection<op={self.op.name!r}, variant={self.variant!r}, args={self.arg_descs}, results={self.result_descs}>"

    @abstractmethod
    def arg_tensor(self, arg: int, *, inplace_tied: bool = False) -> TensorArg: ...

    @abstractmethod
    def arg_optional_tensor(self, arg: int) -> Optional[TensorArg]: ...

    @abstractmethod
    def arg_tensor_list(self, arg: int) -> TensorListArg: ...

    @abstractmethod
    def arg_int(self, arg: int) -> IntArg: ...

    @abstractmethod
    def attr_str(self, arg: int) -> AttrArg: ...

    @abstractmethod
    def attr_int(self, arg: int) -> AttrArg: ...

    @abstractmethod
    def attr_float(self, arg: int) -> AttrArg: ...

    @abstractmethod
    def attr_bool(self, arg: int) -> AttrArg: ...

    def return_tensor(self, t: Tensor) -> TensorArg:
        desc = TensorArg(t)
        self.result_descs.append(desc)
        return desc

    def maybe_return_tensor(self, t: Optional[Tensor]):
        if t is None:
            desc = EmptyOptionalTensorArg()
            self.result_descs.append(desc)
            return desc
        return self.return_tensor(t)

    def return_new_tensor(self, size: Sequence[int], dtype: torch.dtype) -> TensorArg:
        return self.return_tensor(torch.empty(list(size), dtype=dtype, device="meta"))


class EagerKernelSelection(KernelSelection):
    """Selection over concrete call arguments (real, fake or meta tensors)."""

    def __init__(self, op: "CustomOp", args: Sequence[Any]):
        args = list(args)
        # The dispatcher drops trailing arguments that were left at their schema default when it
        # calls a Python implementation; put the defaults back so `select` sees every argument.
        schema_args = _schema_arguments(op)
        for extra in schema_args[len(args):]:
            args.append(extra.default_value if extra.has_default_value() else None)
        super().__init__(op, len(args))
        self.args = args

    def _claim(self, arg: int, expected: type | tuple, what: str):
        assert self.arg_descs[arg] is None, f"Already constrained argument {arg}"
        value = self.args[arg]
        assert isinstance(value, expected), (
            f"Argument type mismatch from Torch for {arg}: Expected {what}, got {type(value)}"
        )
        return value

    def arg_tensor(self, arg: int, *, inplace_tied: bool = False) -> TensorArg:
        desc = TensorArg(self._claim(arg, Tensor, "tensor"))
        self.arg_descs[arg] = desc
        if inplace_tied:
            self.inplace_tied_arg_descs.append(desc)
        return desc

    def arg_optional_tensor(self, arg: int) -> Optional[TensorArg]:
        if arg >= len(self.args):
            self.arg_descs.extend([None] * (arg + 1 - len(self.arg_descs)))
            self.args.extend([None] * (arg + 1 - len(self.args)))
        if self.args[arg] is None:
            self.arg_descs[arg] = EmptyOptionalTensorArg()
            return None
        return self.arg_tensor(arg)

    def arg_tensor_list(self, arg: int) -> TensorListArg:
        desc = TensorListArg(self._claim(arg, list, "list"))
        self.arg_descs[arg] = desc
        return desc

    def arg_int(self, arg: int) -> IntArg:
        desc = IntArg(self._claim(arg, int, "int"))
        self.arg_descs[arg] = desc
        return desc

    def _attr(self, arg: int, expected, what: str) -> AttrArg:
        desc = AttrArg(self._claim(arg, expected, what))
        self.arg_descs[arg] = desc
        return desc

    def attr_str(self, arg: int) -> AttrArg:
        return self._attr(arg, str, "str")

    def attr_int(self, arg: int) -> AttrArg:
        return self._attr(arg, int, "int")

    def attr_float(self, arg: int) -> AttrArg:
        return self._attr(arg, (float, int), "float")

    def attr_bool(self, arg: int) -> AttrArg:
        return self._attr(arg, (bool, int), "bool")

    def attr_optional(self, arg: int) -> AttrArg:
        """An attribute that may be None (e.g. ``ScalarType? out_dtype=None``)."""
        if arg >= len(self.args):
            self.arg_descs.extend([None] * (arg + 1 - len(self.arg_descs)))
            self.args.extend([None] * (arg + 1 - len(self.args)))
        desc = AttrArg(self.args[arg])
        self.arg_descs[arg] = desc
        return desc


# ---------------------------------------------------------------------------------------------
# CustomOp
# ---------------------------------------------------------------------------------------------
class CustomOp(ABC):
    """Subclass, then decorate with ``@CustomOp.register(library=...)`` (base.py:97-168)."""

    @staticmethod
    def register(
        op_class: Optional[Type["CustomOp"]] = None,
        *,
        library: Optional[torch.library.Library] = None,
        dispatch_key: Union[str, Sequence[str], None] = None,
        register_meta: bool = True,
        register_impl: bool = True,
    ) -> Callable:
        if op_class is None:
            return functools.partial(
                CustomOp.register,
                library=library,
                dispatch_key=dispatch_key,
                register_meta=register_meta,
                register_impl=register_impl,
            )
        if library is None:
            from . import ops  # late import: the default library lives with the op definitions

            library = ops.LIBRARY
        instance = op_class(
            library=library, dispatch_key=dispatch_key, register_meta=register_meta, register_impl=register_impl
        )
        return instance.op

    def __init__(self, *, library, dispatch_key, register_meta: bool, register_impl: bool):
        self.name = name = _define_signature_in_library(library, self.signature)
        self.library = library
        self.cache_key_base = f"{library.ns}.{library.kind}::{name}"
        self.op = getattr(getattr(torch.ops, library.ns), name)
        if register_meta:
            library.impl(name, _meta_impl(self), "Meta")
        if register_impl:
            keys = default_dispatch_keys() if dispatch_key is None else (
                [dispatch_key] if isinstance(dispatch_key, str) else list(dispatch_key)
            )
            for k in keys:
                library.impl(name, _impl_trampoline(self), k)
        ALL_CUSTOM_OP_REGS[f"{library.ns}.{name}"] = self

    @property
    @abstractmethod
    def signature(self) -> str:
        """PyTorch schema, e.g. ``my_op(Tensor t) -> Tensor``; ``@UNIQUE@`` in the name is numbered."""

    @abstractmethod
    def select(self, sel: KernelSelection):
        """Describes every argument and declares the result meta tensors."""

    def eager_execute(self, *args):
        """Device implementation.  Must return the op's result."""
        return NotImplemented

    def generate(self, ksel: KernelSelection, kb: Any):
        raise NotImplementedError(
            f"{type(self).__name__}: IR generation is not part of this library; the op runs through "
            "eager_execute only"
        )


def _schema_arguments(op: CustomOp) -> list:
    try:
        return list(op.op.default._schema.arguments)
    except AttributeError:
        return []


def _tensor_args(args) -> list:
    out = []
    for a in args:
        if isinstance(a, torch.Tensor):
            out.append(a)
        elif isinstance(a, (list, tuple)):
            out.extend(t for t in a if isinstance(t, torch.Tensor))
    return out


def _check_one_device(op: CustomOp, args) -> Optional[torch.device]:
    """Every tensor argument (auxiliary ones included: lengths, tables, scales, bias) must live on
    the device of the first one.  The dispatcher picks the CUDA implementation as soon as ONE
    argument is a CUDA tensor, so without this check a host tensor's pointer, or a pointer into
    another GPU's memory, would reach a kernel.  Returns that device (None if there is no tensor)."""
    tensors = _tensor_args(args)
    if not tensors:
        return None
    dev = tensors[0].device
    for t in tensors[1:]:
        torch._check(
            t.device == dev,
            lambda: f"{op.library.ns}.{op.name}: all tensor arguments must be on one device, got {dev} and {t.device}",
        )
    return dev


def _meta_impl(op: CustomOp):
    def meta(*args):
        _check_one_device(op, args)
        sel = EagerKernelSelection(op, args)
        op.select(sel)
        return sel.generate_meta_returns()

    return meta


_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _current_device() -> int:
    return _get_device() if _get_device is not None else torch.cuda.current_device()


def _impl_trampoline(op: CustomOp):
    def handler(*args):
        dev = _check_one_device(op, args)
        if dev is not None and dev.type == "cuda" and dev.index is not None and dev.index != _current_device():
            # launch on the tensors' device, whatever device happens to be current (the reference
            # takes the device from the tensors as well, runtime/op_reg/eager.py:71-100)
            with torch.cuda.device(dev):
                result = op.eager_execute(*args)
        else:
            result = op.eager_execute(*args)
        if result is NotImplemented:
            raise NotImplementedError(
                f"{op.library.ns}.{op.name} has no device implementation (eager_execute returned "
                "NotImplemented) and this library compiles nothing at call time"
            )
        return result

    return handler


_SIGNATURE_RE = re.compile(r"^([^(]+)(\(.+)$")


def _define_signature_in_library(lib: torch.library.Library, signature: str) -> str:
    m = _SIGNATURE_RE.match(signature)
    if not m:
        raise ValueError(f"Expected signature of form `name(...) -> type`. Got: {signature}")
    name, call_args = m.group(1), m.group(2)
    with _CONFIG_LOCK:
        if "@UNIQUE@" in name:
            key = (lib.ns, name)
            _UNIQUE_COUNTERS[key] = _UNIQUE_COUNTERS.get(key, 0) + 1
            name = name.replace("@UNIQUE@", str(_UNIQUE_COUNTERS[key]))
        if (lib.ns, name) in _DEFINED:
            raise RuntimeError(f"Duplicate custom op registration: library={lib.ns}, name={name}")
        lib.define(f"{name}{call_args}")
        _DEFINED.add((lib.ns, name))
    return name
