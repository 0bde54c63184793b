"""Public operators of the ICTC hot path on B200, same names and contracts as the reference's
``ictc_o3/operators.py``: EdgeTensorProduct, PackedGraphMessage, GraphMessage, direction_harmonics,
channel_linear, normalized_silu (+ the symmetric-contraction factories in ``symmetric_contraction``).

Every call lands in ``libictc_b200.so`` through the C ABI; CPU tensors are rejected.
"""
from __future__ import annotations

import torch

from . import _lib
from . import tables

__all__ = [
    "EdgeTensorProduct", "GraphMessage", "PackedGraphMessage", "direction_harmonics",
    "create_symmetric_contraction", "configure_symmetric_contraction",
    "channel_linear", "normalized_silu",
]


def strict_fp32():
    """Ordinary IEEE fp32 everywhere, library GEMMs included (ictc_o3/backends/k100/fp32_policy.py:6-11)."""
    if torch.get_float32_matmul_precision() != "highest" or torch.backends.cuda.matmul.allow_tf32:
        torch.set_float32_matmul_precision("highest")
        torch.backends.cuda.matmul.allow_tf32 = False
    if torch.backends.cudnn.allow_tf32:
        torch.backends.cudnn.allow_tf32 = False


def _degree(value, name):
    if not isinstance(value, int) or isinstance(value, bool) or value < 0:
        raise ValueError(f"{name} must be a nonnegative integer")


def _positive_integer(value, name):
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{name} must be a positive integer")


def _eager(sample):
    """Reject tracing / functorch / autocast contexts (ictc_o3/operators.py:24-32)."""
    strict_fp32()
    from torch.fx.experimental.proxy_tensor import get_proxy_mode
    from torch._subclasses.fake_tensor import is_fake
    if (torch.compiler.is_compiling() or get_proxy_mode() is not None or is_fake(sample)
            or torch._C._are_functorch_transforms_active()
            or torch.is_autocast_enabled(sample.device.type)):
        raise ValueError("Standalone generated TP requires eager execution without autocast")


def _tp_coverage(tp, input_lmax, edge_lmax, allow_live_weight=False):
    from .basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct
    _degree(input_lmax, "input_lmax")
    _degree(edge_lmax, "edge_lmax")
    if not isinstance(tp, EdgeWeightedPathPreservingTensorProduct):
        raise TypeError("Expected an ICTC EdgeWeightedPathPreservingTensorProduct")
    if (tp.channels < 1 or tp.lmax < 0 or not tp.weight.is_cuda
            or tp.weight.dtype != torch.float32 or tp.internal_compute_dtype != torch.float32):
        raise ValueError("Generated TP requires CUDA FP32, internal FP32 and positive channels")
    if tp.weight.requires_grad and not allow_live_weight:
        raise ValueError("TP base coefficients must already be fixed; HP does not freeze learned weights")
    if not tp.paths or any(l1 > input_lmax or l2 > edge_lmax for l1, l2, _ in tp.paths):
        raise ValueError("TP paths must be nonempty and fit the declared input/edge degrees")


def _operand(value, shape, sample, name):
    if not isinstance(value, torch.Tensor) or tuple(value.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}")
    if value.device != sample.device or value.dtype != torch.float32:
        raise ValueError(f"{name} must be FP32 on {sample.device}")


# ------------------------------------------------------------------------------- layout helpers
def _to_ir_mul(flat, channels, widths):
    """mul_ir -> ir_mul for a row buffer made of blocks [count_i*C, m_i] (count folded in widths)."""
    rows, parts, off = flat.shape[0], [], 0
    for count, m in widths:
        w = count * channels * m
        if w:
            parts.append(flat[:, off:off + w].reshape(rows, count, channels, m).transpose(2, 3).reshape(rows, w))
        off += w
    return torch.cat(parts, -1).contiguous() if parts else flat


def _to_mul_ir(flat, channels, widths):
    rows, parts, off = flat.shape[0], [], 0
    for count, m in widths:
        w = count * channels * m
        if w:
            parts.append(flat[:, off:off + w].reshape(rows, count, m, channels).transpose(2, 3).reshape(rows, w))
        off += w
    return torch.cat(parts, -1).contiguous() if parts else flat


class EdgeTensorProduct(torch.nn.Module):
    """Edge-wise TP with fixed base coefficients and live external gates.

    Same buffer contract as the reference (ictc_o3/operators.py:161-340): ``ir_mul`` stores
    [magnetic, channel] inside each degree / path slot, ``mul_ir`` stores [channel, magnetic]; output
    paths stay separate; first, mixed-second and higher autograd are supported; eager execution only.
    ``execution`` is accepted for compatibility ('direct' / 'legacy' select K100 schedules in the
    reference; both map to the same kernels here).
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, layout="ir_mul", execution="direct", _allow_live_weight=False):
        super().__init__()
        _tp_coverage(tp, input_lmax, edge_lmax, _allow_live_weight)
        if layout not in ("ir_mul", "mul_ir"):
            raise ValueError("Edge layout must be 'ir_mul' or 'mul_ir'")
        if execution not in ("direct", "legacy"):
            raise ValueError("Edge execution must be 'direct' or 'legacy'")
        self.tp = tp
        self.input_lmax, self.edge_lmax, self.layout = input_lmax, edge_lmax, layout
        self.execution = execution
        self._allow_live_weight = _allow_live_weight
        out_lmax = max(p[2] for p in tp.paths)
        if [tuple(p) for p in tp.paths] != tables.natural_paths(input_lmax, edge_lmax, out_lmax):
            raise ValueError("Only full natural-parity path sets have compiled kernels "
                             f"(got {list(tp.paths)} for input_lmax={input_lmax}, edge_lmax={edge_lmax})")
        self._spec = _lib.tp_spec(input_lmax, edge_lmax, out_lmax)
        self._unit_version, self._unit = None, False

    @classmethod
    def create(cls, *, input_lmax, edge_lmax, output_lmax=None, channels=64, layout="ir_mul", execution="direct",
               device="cuda"):
        """New FP32 natural-parity TP with unit fixed coefficients (ictc_o3/operators.py:190-215)."""
        _degree(input_lmax, "input_lmax")
        _positive_integer(channels, "channels")
        _degree(edge_lmax, "edge_lmax")
        output_lmax = input_lmax if output_lmax is None else output_lmax
        _degree(output_lmax, "output_lmax")
        if torch.device(device).type != "cuda":
            raise ValueError("Generated edge TP requires a CUDA device")
        from .basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct
        paths = tables.natural_paths(input_lmax, edge_lmax, output_lmax)
        tp = EdgeWeightedPathPreservingTensorProduct(
            channels=channels, lmax=max(input_lmax, edge_lmax, output_lmax),
            allowed_paths=paths, path_policy="full", internal_compute_dtype=torch.float32,
        ).to(device=device, dtype=torch.float32)
        with torch.no_grad():
            tp.weight.fill_(1.)
        tp.weight.requires_grad_(False)
        return cls(tp, input_lmax=input_lmax, edge_lmax=edge_lmax, layout=layout, execution=execution)

    @property
    def paths(self):
        """Immutable external-gate order: (input_l, edge_l, output_l)."""
        return tuple(tuple(path) for path in self.tp.paths)

    @property
    def gate_width(self):
        return self.tp.num_paths * self.tp.channels

    @property
    def output_width(self):
        return sum(self.tp.channels * count * (2 * l + 1) for l, count in self.tp.path_counts_by_l.items())

    def _weight(self):
        """Base coefficients for the kernel, or None when they are all one (checked once per update)."""
        w = self.tp.weight
        version = None if w.is_inference() else w._version
        if version is None or self._unit_version != version:
            self._unit = bool(torch.all(w == 1).item())
            self._unit_version = version
        return None if self._unit else w.detach().contiguous()

    def _in_widths(self):
        return [(1, 2 * l + 1) for l in range(self.input_lmax + 1)]

    def _out_widths(self):
        return [(self.tp.path_counts_by_l.get(l, 0), 2 * l + 1) for l in range(self.tp.lmax + 1)]

    def pack_input(self, blocks):
        """Pack {l: [E,C,2l+1]} using this operator's layout."""
        if set(blocks) != set(range(self.input_lmax + 1)):
            raise ValueError("Input blocks must cover every declared degree")
        rows, parts = blocks[0].shape[0], []
        for l in range(self.input_lmax + 1):
            block = blocks[l]
            _operand(block, (rows, self.tp.channels, 2 * l + 1), self.tp.weight, f"blocks[{l}]")
            if self.layout == "ir_mul":
                block = block.transpose(1, 2)
            parts.append(block.reshape(rows, self.tp.channels * (2 * l + 1)))
        return torch.cat(parts, -1).contiguous()

    def unpack_output(self, output):
        """Return {l: [E,C*path_count_l,2l+1]} in the ICTC convention."""
        rows = output.shape[0]
        _operand(output, (rows, self.output_width), self.tp.weight, "output")
        result, offset = {}, 0
        for l in range(self.tp.lmax + 1):
            count, width = self.tp.path_counts_by_l.get(l, 0), 2 * l + 1
            value = output[:, offset:offset + count * self.tp.channels * width]
            if self.layout == "ir_mul":
                value = value.reshape(rows, count, width, self.tp.channels).transpose(2, 3)
            result[l] = value.reshape(rows, count * self.tp.channels, width)
            offset += count * self.tp.channels * width
        return result

    def forward(self, features, harmonics, gates):
        """features [E,C*(L_in+1)^2], harmonics [E,(L_edge+1)^2], gates [E,P*C] or [E,P,C]."""
        _tp_coverage(self.tp, self.input_lmax, self.edge_lmax, self._allow_live_weight)
        _eager(features)
        if features.ndim != 2:
            raise ValueError("features must be a flat two-dimensional row buffer")
        rows, c = features.shape[0], self.tp.channels
        _operand(features, (rows, c * (self.input_lmax + 1) ** 2), self.tp.weight, "features")
        _operand(harmonics, (rows, (self.edge_lmax + 1) ** 2), self.tp.weight, "harmonics")
        _operand(gates, (rows, self.gate_width) if gates.ndim == 2 else (rows, self.tp.num_paths, c),
                 self.tp.weight, "gates")
        if rows == 0:
            empty = features[:, :1] * harmonics[:, :1] * gates.reshape(0, self.gate_width)[:, :1]
            return empty.expand(0, self.output_width)
        from .ops.tensor_product import TpCall, tensor_product
        if self.layout == "mul_ir":
            features = _to_ir_mul(features, c, self._in_widths())
        call = TpCall(self._spec, c, self._weight(), None, None)
        output = tensor_product(features.contiguous(), harmonics.contiguous(),
                                gates.reshape(rows, self.gate_width).contiguous(), call)
        if self.layout == "mul_ir":
            output = _to_mul_ir(output, c, self._out_widths())
        return output


class PackedGraphMessage(torch.nn.Module):
    """Packed gather / TP / scatter-sum without dictionary layout round trips.

    Input/output layout matches EdgeTensorProduct(layout='ir_mul') (ictc_o3/operators.py:343-409).
    The reduction is always the receiver-CSR, atomic-free one; ``reduction`` ('atomic' / 'csr') and
    the K100 tuning options are accepted and ignored.
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, cartesian_schedule='native', reduction='atomic',
                 edge_chunk_size=65536, topology_backend='native', csr_accumulator_limit=None,
                 csr_slice_search=False, geometry_schedule='auto'):
        super().__init__()
        if cartesian_schedule != 'native':
            raise ValueError('Only the original ICTC basis is supported; the experimental STF-coordinate schedule is retired')
        if reduction not in ('atomic', 'csr'):
            raise ValueError('Packed graph reduction must be atomic or csr')
        if topology_backend not in ('native', 'device'):
            raise ValueError('Topology backend must be native or device')
        if csr_accumulator_limit is not None and (not isinstance(csr_accumulator_limit, int)
                                                  or isinstance(csr_accumulator_limit, bool) or csr_accumulator_limit < 1):
            raise ValueError('CSR accumulator limit must be a positive integer or None')
        if not isinstance(csr_slice_search, bool):
            raise ValueError('csr_slice_search must be a bool')
        if geometry_schedule not in ('auto', 'native', 'streamed'):
            raise ValueError('geometry_schedule must be auto, native or streamed')
        if not isinstance(edge_chunk_size, int) or isinstance(edge_chunk_size, bool) or edge_chunk_size < 1:
            raise ValueError('edge_chunk_size must be a positive integer')
        self.edge = EdgeTensorProduct(tp, input_lmax=input_lmax, edge_lmax=edge_lmax)
        self.cartesian_schedule, self.reduction, self.edge_chunk_size = cartesian_schedule, reduction, edge_chunk_size
        self._topology_key, self._topology = None, None

    @classmethod
    def create(cls, *, channels=64, input_lmax=3, edge_lmax=3, output_lmax=None, device='cuda', **kwargs):
        edge = EdgeTensorProduct.create(channels=channels, input_lmax=input_lmax, edge_lmax=edge_lmax,
                                        output_lmax=output_lmax, device=device)
        return cls(edge.tp, input_lmax=input_lmax, edge_lmax=edge_lmax, **kwargs)

    @property
    def tp(self):
        return self.edge.tp

    @property
    def output_width(self):
        return self.edge.output_width

    @property
    def gate_width(self):
        return self.edge.gate_width

    def topology(self, src, dst, num_nodes):
        """CSR pair of a live edge list; rebuilt when the index tensors change."""
        from .ops.topology import Topology
        key = (src.data_ptr(), src._version, dst.data_ptr(), dst._version, src.numel(), num_nodes)
        if key != self._topology_key:
            self._topology, self._topology_key = Topology(src, dst, num_nodes), key
        return self._topology

    def forward(self, features, harmonics, gates, src, dst, mask=None):
        _eager(features)
        _tp_coverage(self.tp, self.edge.input_lmax, self.edge.edge_lmax)
        if features.ndim != 2:
            raise ValueError('Expected a flat two-dimensional packed node buffer')
        n, e, c = features.shape[0], src.numel(), self.tp.channels
        _operand(features, (n, c * (self.edge.input_lmax + 1) ** 2), self.tp.weight, 'features')
        _operand(harmonics, (e, (self.edge.edge_lmax + 1) ** 2), self.tp.weight, 'harmonics')
        _operand(gates, (e, self.gate_width) if gates.ndim == 2 else (e, self.tp.num_paths, c), self.tp.weight, 'gates')
        for name, value in (('src', src), ('dst', dst)):
            if value.ndim != 1 or value.numel() != e or value.device != features.device or value.dtype != torch.int64:
                raise ValueError(f'{name} must be an int64 CUDA vector of valid node indices')
        if mask is not None:
            if mask.requires_grad or tuple(mask.shape) not in ((e,), (e, 1)):
                raise ValueError('Mask must be fixed [E] or [E,1]')
            _operand(mask, mask.shape, self.tp.weight, 'mask')
            mask = mask.reshape(e).contiguous()
        from .ops.tensor_product import TpCall, tensor_product
        call = TpCall(self.edge._spec, c, self.edge._weight(), mask, self.topology(src, dst, n))
        return tensor_product(features.contiguous(), harmonics.contiguous(),
                              gates.reshape(e, self.gate_width).contiguous(), call)


class GraphMessage(torch.nn.Module):
    """Gather / TP / gate / scatter with repeated destinations and live inputs, dictionary I/O.

    features {l:[N,C,2l+1]}, harmonics {l:[E,1,2l+1]}, gates [E,P*C] -> {l:[N,count_l*C,2l+1]}
    (ictc_o3/operators.py:412-468).  ``layout`` ('packed' / 'fused_pack' / 'canonical') and
    ``reduction`` select K100 schedules in the reference; here they are accepted and the kernels
    always work on ir_mul rows with the receiver-CSR reduction.
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, layout="packed", edge_chunk_size=65536, reduction="auto",
                 cartesian_schedule="native"):
        super().__init__()
        _tp_coverage(tp, input_lmax, edge_lmax)
        if layout not in ("packed", "fused_pack", 'canonical'):
            raise ValueError("Graph layout must be packed, fused_pack or canonical")
        if reduction not in ("auto", "atomic", "csr"):
            raise ValueError("Graph reduction must be auto, atomic or csr")
        if cartesian_schedule != 'native':
            raise ValueError('Only the original ICTC basis is supported; the experimental STF-coordinate schedule is retired')
        if not isinstance(edge_chunk_size, int) or isinstance(edge_chunk_size, bool) or edge_chunk_size < 1:
            raise ValueError("edge_chunk_size must be a positive integer")
        self.tp, self.input_lmax, self.edge_lmax = tp, input_lmax, edge_lmax
        self.layout, self.edge_chunk_size = layout, edge_chunk_size
        self._packed = PackedGraphMessage(tp, input_lmax=input_lmax, edge_lmax=edge_lmax)

    def forward(self, features, harmonics, gates, src, dst, mask=None):
        _tp_coverage(self.tp, self.input_lmax, self.edge_lmax)
        if set(features) != set(range(self.input_lmax + 1)) or set(harmonics) != set(range(self.edge_lmax + 1)):
            raise ValueError("Degree dictionaries must cover declared input/edge degrees")
        _eager(features[0])
        n, e, c = features[0].shape[0], src.numel(), self.tp.channels
        for l, value in features.items():
            _operand(value, (n, c, 2 * l + 1), self.tp.weight, f"features[{l}]")
        for l, value in harmonics.items():
            _operand(value, (e, 1, 2 * l + 1), self.tp.weight, f"harmonics[{l}]")
        _operand(gates, (e, self.tp.num_paths * c), self.tp.weight, "gates")
        edge = self._packed.edge
        x = torch.cat([features[l].transpose(1, 2).reshape(n, -1) for l in range(self.input_lmax + 1)], -1)
        sh = torch.cat([harmonics[l].reshape(e, 2 * l + 1) for l in range(self.edge_lmax + 1)], -1)
        out = self._packed(x, sh, gates, src, dst, mask)
        return edge.unpack_output(out)


def direction_harmonics(directions, lmax, *, policy="auto"):
    """Component-normalized Cartesian harmonics: list of [E,2l+1] unit-direction blocks.

    Input is [E,3] unit vectors on a CUDA device (callers normalise their displacements and
    differentiate through that).  ``policy`` is accepted for compatibility; there is one path.
    (ictc_o3/operators.py:471-490)
    """
    _degree(lmax, "lmax")
    if directions.ndim != 2 or directions.shape[1] != 3:
        raise ValueError("directions must have shape [E,3]")
    if policy not in ("auto", "generated", "reference"):
        raise ValueError("Harmonic policy must be auto, generated or reference")
    if not directions.is_cuda or directions.dtype != torch.float32:
        raise ValueError("Generated harmonics require eager CUDA FP32 and no autocast")
    if lmax > tables.TABLE_LMAX:
        raise ValueError(f"direction harmonics are compiled up to lmax {tables.TABLE_LMAX}")
    from .ops.harmonics import harmonics_flat
    output = harmonics_flat(directions, lmax)
    return list(output.split([2 * l + 1 for l in range(lmax + 1)], -1))


def channel_linear(features, weight, bias=None):
    """Shared-weight channel GEMM: [*,Cin,m] x [Cout,Cin] -> [*,Cout,m] (ictc_o3/operators.py:609-628)."""
    strict_fp32()
    if features.ndim < 2 or weight.ndim != 2 or features.shape[-2] != weight.shape[1]:
        raise ValueError("Expected features [*,Cin,m] and weight [Cout,Cin]")
    if features.device != weight.device or features.dtype != weight.dtype:
        raise ValueError("Features and weights must share device and dtype")
    if bias is not None:
        if features.shape[-1] != 1:
            raise ValueError("Channel bias is allowed only for the scalar angular block")
        if bias.shape != (weight.shape[0],) or bias.device != weight.device or bias.dtype != weight.dtype:
            raise ValueError("bias must match output channel count, device and dtype")
    angular = features.movedim(-2, -1).contiguous()
    output = torch.nn.functional.linear(angular.reshape(-1, weight.shape[1]), weight, bias)
    return output.reshape(*angular.shape[:-1], weight.shape[0]).movedim(-1, -2)


def normalized_silu(features, scale=1.0):
    """SiLU times a fixed scale (ictc_o3/operators.py:631-636)."""
    if not isinstance(scale, (int, float)) or isinstance(scale, bool):
        raise TypeError("scale must be a fixed numeric scalar")
    return torch.nn.functional.silu(features) * float(scale)


def create_symmetric_contraction(**kwargs):
    from .symmetric_contraction import create_symmetric_contraction as impl
    return impl(**kwargs)


def configure_symmetric_contraction(module, **kwargs):
    from .symmetric_contraction import configure_symmetric_contraction as impl
    return impl(module, **kwargs)
