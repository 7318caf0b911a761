"""A small stand-in for the parts of DaCe that DaCeML's ONNX library nodes live in.

The reference builds an SDFG whose single state holds ``ONNX<Op>`` library nodes joined to
AccessNodes by memlets, expands every library node, and lets DaCe generate code
(``daceml/onnx/onnx_importer.py:197-338``, ``daceml/util/utils.py:156-202``).  DaCe is not part of
this build, so this module provides the same shapes with the same method names -- ``SDFG``,
``SDFGState``, ``AccessNode``, ``Memlet``, ``add_array``, ``add_edge``, ``make_array_memlet``,
``expand_library_nodes`` -- and replaces code generation with a launch plan: an expanded node is a
:class:`KernelTasklet` whose callable enqueues CUDA kernels on the current stream.
"""
import collections
from typing import Callable, Dict, List, Optional

import numpy as np
import os

import torch

_NP_TO_TORCH = {
    np.dtype("float16"): torch.float16, np.dtype("float32"): torch.float32, np.dtype("float64"): torch.float64,
    np.dtype("int32"): torch.int32, np.dtype("int64"): torch.int64, np.dtype("bool"): torch.bool,
    np.dtype("int8"): torch.int8, np.dtype("uint8"): torch.uint8,
}


def to_torch_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        return dtype
    return _NP_TO_TORCH[np.dtype(dtype)]


class Data:
    """Array descriptor: the counterpart of ``dace.data.Array`` (shape, dtype, transient flag)."""

    def __init__(self, shape, dtype, transient=False):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = to_torch_dtype(dtype)
        self.transient = transient
        # name of the array whose storage this one shares (a reshape of it); the counterpart of ``dace.data.View``
        self.view_of = None

    @property
    def strides(self):
        out, acc = [], 1
        for s in reversed(self.shape):
            out.append(acc)
            acc *= s
        return tuple(reversed(out))

    def total_size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def __repr__(self):
        return f"Data({list(self.shape)}, {self.dtype}{', transient' if self.transient else ''})"


class Memlet:
    def __init__(self, data):
        self.data = data


class Node:
    pass


class AccessNode(Node):
    def __init__(self, data):
        self.data = data

    def __repr__(self):
        return f"AccessNode({self.data})"


class KernelTasklet(Node):
    """What an expansion returns here: a callable that launches kernels.

    ``fn(inputs, outputs)`` receives dictionaries connector -> torch tensor.  Inside real DaCe the
    same role is played by a CPP tasklet that calls the C ABI (the pattern of
    ``daceml/onnx/op_implementations/cudnn_implementations.py:384-401``)."""

    def __init__(self, label, fn: Callable[[Dict[str, torch.Tensor], Dict[str, torch.Tensor]], None], kernels=()):
        self.label = label
        self.fn = fn
        self.kernels = tuple(kernels)

    def __repr__(self):
        return f"KernelTasklet({self.label})"


Edge = collections.namedtuple("Edge", ["src", "src_conn", "dst", "dst_conn", "data"])


class SDFGState:
    def __init__(self, sdfg, label="state"):
        self.parent = sdfg
        self.label = label
        self._nodes: List[Node] = []
        self._edges: List[Edge] = []

    # -- construction ------------------------------------------------------------------------
    def add_node(self, node):
        if node not in self._nodes:
            self._nodes.append(node)
        return node

    def add_access(self, name):
        if name not in self.parent.arrays:
            raise KeyError(f"array '{name}' is not defined in SDFG '{self.parent.name}'")
        return self.add_node(AccessNode(name))

    add_read = add_access
    add_write = add_access

    def add_edge(self, src, src_conn, dst, dst_conn, memlet):
        self.add_node(src)
        self.add_node(dst)
        # library nodes grow connectors on demand, like LibraryNode.add_in_connector in DaCe
        if src_conn is not None and hasattr(src, "add_out_connector"):
            src.add_out_connector(src_conn)
        if dst_conn is not None and hasattr(dst, "add_in_connector"):
            dst.add_in_connector(dst_conn)
        e = Edge(src, src_conn, dst, dst_conn, memlet)
        self._edges.append(e)
        return e

    def remove_node(self, node):
        self._nodes.remove(node)
        self._edges = [e for e in self._edges if e.src is not node and e.dst is not node]

    def remove_edge(self, edge):
        self._edges.remove(edge)

    # -- queries -----------------------------------------------------------------------------
    def nodes(self):
        return list(self._nodes)

    def edges(self):
        return list(self._edges)

    def in_edges(self, node):
        return [e for e in self._edges if e.dst is node]

    def out_edges(self, node):
        return [e for e in self._edges if e.src is node]

    def in_edges_by_connector(self, node, conn):
        return (e for e in self._edges if e.dst is node and e.dst_conn == conn)

    def out_edges_by_connector(self, node, conn):
        return (e for e in self._edges if e.src is node and e.src_conn == conn)

    def replace_node(self, old, new):
        """Swaps a library node for its expansion, keeping every edge."""
        idx = self._nodes.index(old)
        self._nodes[idx] = new
        self._edges = [Edge(new if e.src is old else e.src, e.src_conn, new if e.dst is old else e.dst, e.dst_conn,
                            e.data) for e in self._edges]

    def topological_compute_nodes(self):
        """Non-access nodes ordered so that producers of an array come before its consumers."""
        compute = [n for n in self._nodes if not isinstance(n, AccessNode)]
        root = self.parent.root_of  # a view is written by whoever writes the array it aliases
        writers = collections.defaultdict(list)
        for n in compute:
            for e in self.out_edges(n):
                writers[root(e.data.data)].append(n)
        deps = {id(n): set() for n in compute}
        for n in compute:
            for e in self.in_edges(n):
                for w in writers.get(root(e.data.data), ()):
                    if w is not n:
                        deps[id(n)].add(id(w))
        order, done, pending = [], set(), list(compute)
        while pending:
            progressed = False
            for n in list(pending):
                if deps[id(n)] <= done:
                    order.append(n)
                    done.add(id(n))
                    pending.remove(n)
                    progressed = True
            if not progressed:
                raise ValueError(f"cycle in state '{self.label}'")
        return order


class SDFG:
    def __init__(self, name):
        self.name = name
        self.arrays: Dict[str, Data] = {}
        self._states: List[SDFGState] = []
        # constants bound at build time (weights), name -> tensor; the importer's ``weights`` dict
        self.constants: Dict[str, torch.Tensor] = {}

    def add_array(self, name, shape, dtype, transient=False):
        if name in self.arrays:
            raise NameError(f"array '{name}' already exists")
        self.arrays[name] = Data(shape, dtype, transient)
        return name, self.arrays[name]

    def add_transient(self, name, shape, dtype):
        return self.add_array(name, shape, dtype, transient=True)

    def add_scalar(self, name, dtype, transient=False):
        return self.add_array(name, (), dtype, transient)

    def add_datadesc(self, name, desc):
        self.arrays[name] = desc
        return name

    def add_constant(self, name, tensor):
        self.constants[name] = tensor
        if name not in self.arrays:
            self.add_array(name, tensor.shape, tensor.dtype)

    def root_of(self, name):
        """The array that owns the storage ``name`` refers to (``name`` itself unless it is a view)."""
        seen = set()
        while name in self.arrays and self.arrays[name].view_of is not None and name not in seen:
            seen.add(name)
            name = self.arrays[name].view_of
        return name

    def add_state(self, label=None):
        st = SDFGState(self, label or f"state_{len(self._states)}")
        self._states.append(st)
        return st

    def states(self):
        return list(self._states)

    def make_array_memlet(self, name):
        if name not in self.arrays:
            raise KeyError(name)
        return Memlet(name)

    def all_nodes_recursive(self):
        for st in self._states:
            for n in st.nodes():
                yield n, st

    def expand_library_nodes(self, recursive=True):
        """Expands every library node with its selected implementation (DaCe's method of the same name)."""
        from daceml_b200.util.utils import expand_onnx_nodes
        expand_onnx_nodes(self)

    def compile(self):
        self.expand_library_nodes()
        return CompiledSDFG(self)

    def __call__(self, **kwargs):
        return self.compile()(**kwargs)


NVTX_RANGES = os.environ.get("DACEML_B200_NVTX", "0") == "1"


class CompiledSDFG:
    """The launch plan of an expanded SDFG: tasklets in dependency order plus its transients.

    ``__call__`` binds caller tensors by array name (numpy arrays are staged through the GPU and
    copied back, torch CUDA tensors are used in place), allocates ``__return*`` arrays if the
    caller did not pass them, and enqueues every tasklet on the current CUDA stream."""

    def __init__(self, sdfg: SDFG, device: Optional[torch.device] = None):
        self.sdfg = sdfg
        self.device = device
        self.plan = []
        for st in sdfg.states():
            for n in st.topological_compute_nodes():
                if not isinstance(n, KernelTasklet):
                    raise RuntimeError(f"node {n} was not expanded")
                ins = {e.dst_conn: e.data.data for e in st.in_edges(n)}
                outs = {e.src_conn: e.data.data for e in st.out_edges(n)}
                self.plan.append((n, ins, outs))
        self._transients = {}
        if device is not None or torch.cuda.is_available():
            self.allocate_transients()

    def allocate_transients(self):
        """Allocates every transient of the SDFG (intermediate tensors and the scratch of expansions) now, so that no
        launch allocates: a first call may then run under CUDA-graph capture."""
        dev = self._device()
        for name, desc in self.sdfg.arrays.items():
            if desc.transient and desc.view_of is None and name not in self._transients and name not in self.sdfg.constants:
                self._transients[name] = torch.empty(desc.shape, dtype=desc.dtype, device=dev)

    def _device(self):
        if self.device is None:
            if not torch.cuda.is_available():
                raise RuntimeError("daceml_b200 needs a CUDA device (B200); there is no CPU path")
            self.device = torch.device("cuda", torch.cuda.current_device())
        return self.device

    def kernel_names(self):
        return [k for t, _, _ in self.plan for k in t.kernels]

    def check_status(self, synchronize=True):
        """Raises if a kernel on this SDFG's device recorded a problem (bad Gather index, a wait that ran out) since
        the last check.  Kernels never stop the process; they leave a code in the context's status word."""
        from daceml_b200 import lib as L
        dev = self._device()
        if synchronize:
            torch.cuda.synchronize(dev)
        code = L.get_context(dev).device_status()
        if code != 0:
            raise L.B200Error(L.ERR_DEVICE, "device status 0x%x after running SDFG '%s'" % (code & 0xffffffff, self.sdfg.name))

    def __call__(self, **kwargs):
        dev = self._device()
        bound: Dict[str, torch.Tensor] = {}
        copy_back = []
        for name, val in kwargs.items():
            if name not in self.sdfg.arrays:
                raise KeyError(f"'{name}' is not an array of SDFG '{self.sdfg.name}'")
            desc = self.sdfg.arrays[name]
            if isinstance(val, np.ndarray):
                t = torch.from_numpy(np.ascontiguousarray(val)).to(dev)
                copy_back.append((name, val, t))
            elif isinstance(val, torch.Tensor):
                t = val if val.is_cuda else val.to(dev)
                if not val.is_cuda:
                    copy_back.append((name, val, t))
                if not t.is_contiguous():
                    t = t.contiguous()  # the reference's dispatchers guard inputs the same way
            else:
                t = torch.tensor(val, dtype=desc.dtype, device=dev)
            if tuple(t.shape) != desc.shape or t.dtype != desc.dtype:
                raise ValueError(f"argument '{name}' is {tuple(t.shape)} {t.dtype}, expected {desc.shape} {desc.dtype}")
            bound[name] = t
        for name, t in self.sdfg.constants.items():
            if name not in bound:
                if not t.is_cuda:
                    t = self.sdfg.constants[name] = t.to(dev).contiguous()
                bound[name] = t
        returns = []
        views = []
        for name, desc in self.sdfg.arrays.items():
            if name in bound:
                continue
            if desc.view_of is not None:
                views.append(name)
                continue
            if desc.transient:
                t = self._transients.get(name)
                if t is None:
                    t = self._transients[name] = torch.empty(desc.shape, dtype=desc.dtype, device=dev)
                bound[name] = t
            elif name.startswith("__return"):
                bound[name] = torch.empty(desc.shape, dtype=desc.dtype, device=dev)
                returns.append(name)
            else:
                raise TypeError(f"missing argument '{name}' for SDFG '{self.sdfg.name}'")
        for name in views:  # same storage, other shape (every tensor here is contiguous)
            bound[name] = bound[self.sdfg.root_of(name)].view(self.sdfg.arrays[name].shape)
        if NVTX_RANGES:
            # one named range per SDFG call and per expanded node, as the reference's profiling helpers bracket their
            # functions (daceml/testing/profiling/event_profiler.py:87-120); off unless DACEML_B200_NVTX=1
            torch.cuda.nvtx.range_push(self.sdfg.name)
        for tasklet, ins, outs in self.plan:
            if NVTX_RANGES:
                torch.cuda.nvtx.range_push(tasklet.label)
            tasklet.fn({c: bound[a] for c, a in ins.items()}, {c: bound[a] for c, a in outs.items()})
            if NVTX_RANGES:
                torch.cuda.nvtx.range_pop()
        if NVTX_RANGES:
            torch.cuda.nvtx.range_pop()
        written = {a for _, _, outs in self.plan for a in outs.values()}
        written |= {self.sdfg.root_of(a) for a in written}
        for name, host, devt in copy_back:
            if name not in written and self.sdfg.root_of(name) not in written:
                continue  # a pure input: nothing to bring back
            if isinstance(host, np.ndarray):
                host[...] = devt.cpu().numpy()
            else:
                host.copy_(devt)
        if not returns:
            return None
        # '__return', '__return_0', ... '__return_10': by number, not by string ('__return_10' < '__return_2')
        outs = [bound[n] for n in sorted(returns, key=lambda n: (int(n.rsplit("_", 1)[1]) if n.rsplit("_", 1)[1].isdigit() else -1, n))]
        if any(isinstance(v, np.ndarray) for v in kwargs.values()):
            outs = [o.cpu().numpy() for o in outs]
        return outs[0] if len(outs) == 1 else tuple(outs)
