"""Load plans: which rows of which tensor live on which logical device.

Host-side mirror of the reference's placement planner (src/format/load_plan.rs:6-45 types,
:158-350 `build_load_plan`, :352-590 `LoadPlan::validate` / `used_bytes`) over the segment
index its package exporter derives from a GGUF (src/format/ggufrs.rs:575-735: one Shared
segment for tensors outside `blk.N.`, one Layer segment per block, tensors inside a segment
sorted by name bytes and laid out at `general.alignment`).  The plan is metadata only; a
rank executes its part with `execute_plan`, which turns every placement on its device into
one row-sliced `rmi_weight_upload_gguf` call, so the reference's own placement rules
select the multi-GPU row ranges.  The binary `.ggufrs` container itself is not read here:
the index is rebuilt from the source GGUF with the exporter's layout rules.

The planner walks devices in order and never goes back: shared tensors go whole to the
primary device; LayerSplit then places whole layer segments, TensorSplit fills the current
device with as many complete quantized rows as fit and moves on (a tensor is cut only
where a device fills up).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

from . import gguf as _gguf

SHARED, LAYER, COMPONENT = 1, 2, 3          # SegmentKind, src/format/ggufrs.rs:29-33
LAYER_SPLIT, TENSOR_SPLIT = "LayerSplit", "TensorSplit"
WHOLE = None                                # PlacementSlice::Whole; Rows is a (start, end) tuple

# src/core/tensor.rs type_traits: (block elements, block bytes)
TYPE_TRAITS = {0: (1, 4), 1: (1, 2), 2: (32, 18), 8: (32, 34), 12: (256, 144), 14: (256, 210)}


class PlanError(ValueError):
    """GgufrsError::InvalidPlan"""


class CapacityExceeded(PlanError):
    def __init__(self, device_id, required, available, context):
        super().__init__(f"device {device_id} capacity exceeded for {context}: required {required}, "
                         f"available {available}")
        self.device_id, self.required, self.available = device_id, required, available


class UnsplittableTensor(PlanError):
    def __init__(self, tensor, row_bytes, remaining, reason):
        super().__init__(f"tensor {tensor} cannot be split ({reason}); row bytes {row_bytes}, remaining {remaining}")
        self.tensor, self.row_bytes, self.remaining, self.reason = tensor, row_bytes, remaining, reason


@dataclass(frozen=True)
class TensorRecord:
    component_id: int
    segment_id: int
    name: str
    dims: tuple
    ggml_type: int
    segment_offset: int
    byte_len: int


@dataclass(frozen=True)
class Segment:
    id: int
    component_id: int
    kind: int
    layer: int | None


@dataclass(frozen=True)
class LogicalDevice:
    id: str
    capacity: int


@dataclass(frozen=True)
class Placement:
    component_id: int
    segment_id: int
    tensor_name: str
    slice: tuple | None
    segment_byte_range: tuple
    device_id: str


def layer_index(name: str):
    """src/format/ggufrs.rs:379-386"""
    if not name.startswith("blk."):
        return None
    index, dot, suffix = name[4:].partition(".")
    if not dot or not suffix or not index.isdigit():
        return None
    return int(index)


@dataclass
class PackageIndex:
    """The part of a package index the planner reads: segments and tensor records of the
    selected components, in package order."""
    segments: list = field(default_factory=list)
    tensors: list = field(default_factory=list)
    components: list = field(default_factory=lambda: [0])

    @classmethod
    def from_tensor_table(cls, table, block_count: int, alignment: int = 32, component_id: int = 0):
        """table: [(name, dims, ggml_type)] of an LLM GGUF."""
        groups = [(SHARED, None, [])] + [(LAYER, i, []) for i in range(block_count)]
        for name, dims, gtype in table:
            layer = layer_index(name)
            if layer is not None and layer >= block_count:
                raise PlanError(f"tensor {name} layer {layer} is outside block count {block_count}")
            groups[0 if layer is None else layer + 1][2].append((name, tuple(int(d) for d in dims), int(gtype)))
        idx = cls(components=[component_id])
        for kind, layer, tensors in groups:
            if not tensors:
                raise PlanError(f"{'layer %d' % layer if layer is not None else 'Shared'} segment has no tensors")
            seg = Segment(len(idx.segments), component_id, kind, layer)
            cursor = 0
            for name, dims, gtype in sorted(tensors, key=lambda t: t[0].encode()):
                be, bb = TYPE_TRAITS[gtype]
                n_el = 1
                for d in dims:
                    n_el *= d
                if n_el % be:
                    raise PlanError(f"tensor {name} dimensions/type do not form complete GGML blocks")
                off = (cursor + alignment - 1) // alignment * alignment
                nb = n_el // be * bb
                idx.tensors.append(TensorRecord(component_id, seg.id, name, dims, gtype, off, nb))
                cursor = off + nb
            idx.segments.append(seg)
        return idx

    @classmethod
    def from_gguf_file(cls, path: str):
        g = _gguf.GGUFFile(path)
        arch = g.metadata["general.architecture"]
        table = [(n, d, t) for n, (d, t, _) in g.tensors.items()]
        return cls.from_tensor_table(table, int(g.metadata[f"{arch}.block_count"]),
                                     int(g.metadata.get("general.alignment", 32)))

    def segment(self, segment_id):
        return next((s for s in self.segments if s.id == segment_id), None)


def row_layout(rec: TensorRecord):
    """src/format/load_plan.rs:57-92 -> (row_count, row_bytes)"""
    if not rec.dims:
        raise PlanError(f"{rec.name} has rank zero")
    row_elements = rec.dims[0]
    row_count = 1
    for d in rec.dims[1:]:
        row_count *= d
    be, bb = TYPE_TRAITS[rec.ggml_type]
    if row_elements == 0 or row_elements % be:
        raise UnsplittableTensor(rec.name, 0, [], "row element count is not divisible by quantization block size")
    row_bytes = row_elements // be * bb
    if row_count * row_bytes != rec.byte_len:
        raise PlanError(f"{rec.name} row layout does not match byte_len {rec.byte_len}")
    return row_count, row_bytes


def _validate_devices(devices, primary):
    if not devices:
        raise PlanError("load plan requires at least one logical device")
    seen = set()
    for d in devices:
        if not d.id:
            raise PlanError("logical device id must not be empty")
        if d.id in seen:
            raise PlanError(f"duplicate logical device id {d.id!r}")
        seen.add(d.id)
    return _device_index(devices, primary)


def _device_index(devices, dev_id):
    for i, d in enumerate(devices):
        if d.id == dev_id:
            return i
    raise PlanError(f"unknown logical device {dev_id!r}")


def _selected_components(index, component_ids):
    if len(set(component_ids)) != len(component_ids):
        raise PlanError("selected component ids must be unique")
    selected = [c for c in index.components if c in set(component_ids)]
    for c in component_ids:
        if c not in selected:
            raise PlanError(f"unknown component id {c}")
    return selected


@dataclass
class LoadPlan:
    component_ids: list
    devices: list
    primary_device: str
    policy: str
    placements: list

    def used_bytes(self, device_id: str) -> int:
        _device_index(self.devices, device_id)
        return sum(p.segment_byte_range[1] - p.segment_byte_range[0] for p in self.placements
                   if p.device_id == device_id)

    def rows_on(self, tensor_name: str, device_id: str):
        """[(row_start, row_end)] of the tensor's placements on one device (Whole = all rows)."""
        return [p.slice for p in self.placements if p.tensor_name == tensor_name and p.device_id == device_id]

    def validate(self, index: PackageIndex) -> None:
        """src/format/load_plan.rs:352-580"""
        _validate_devices(self.devices, self.primary_device)
        if _selected_components(index, self.component_ids) != list(self.component_ids):
            raise PlanError("component ids are not in package order")
        selected = set(self.component_ids)
        by_key = {(r.component_id, r.segment_id, r.name): r for r in index.tensors}
        for p in self.placements:
            if p.component_id not in selected:
                raise PlanError(f"placement references unselected component {p.component_id}")
            _device_index(self.devices, p.device_id)
            rec = by_key.get((p.component_id, p.segment_id, p.tensor_name))
            if rec is None:
                raise PlanError(f"placement references unknown tensor {p.tensor_name}")
            lo, hi = rec.segment_offset, rec.segment_offset + rec.byte_len
            s, e = p.segment_byte_range
            if s > e or s < lo or e > hi:
                raise PlanError(f"tensor {p.tensor_name} placement range {s}..{e} is outside {lo}..{hi}")
        layer_devices = {}
        for rec in index.tensors:
            if rec.component_id not in selected:
                continue
            seg = index.segment(rec.segment_id)
            if seg is None:
                raise PlanError(f"tensor {rec.name} references unknown segment {rec.segment_id}")
            row_count, row_bytes = row_layout(rec)
            whole = (rec.segment_offset, rec.segment_offset + rec.byte_len)
            ranges = []
            for p in self.placements:
                if (p.component_id, p.segment_id, p.tensor_name) != (rec.component_id, rec.segment_id, rec.name):
                    continue
                if seg.kind != LAYER and p.device_id != self.primary_device:
                    raise PlanError(f"tensor {rec.name} must be on primary device {self.primary_device!r}")
                if self.policy == LAYER_SPLIT and p.slice is not WHOLE:
                    raise PlanError(f"LayerSplit placement for tensor {rec.name} is not whole")
                if self.policy == LAYER_SPLIT and seg.kind == LAYER:
                    if layer_devices.setdefault(seg.id, p.device_id) != p.device_id:
                        raise PlanError(f"layer segment {seg.id} spans devices")
                if p.slice is WHOLE:
                    if tuple(p.segment_byte_range) != whole:
                        raise PlanError(f"whole placement for tensor {rec.name} has byte range "
                                        f"{p.segment_byte_range}, expected {whole}")
                    ranges.append((0, row_count))
                else:
                    start, end = p.slice
                    if start >= end or end > row_count:
                        raise PlanError(f"tensor {rec.name} has invalid row range {start}..{end} of {row_count}")
                    expect = (rec.segment_offset + start * row_bytes, rec.segment_offset + end * row_bytes)
                    if tuple(p.segment_byte_range) != expect:
                        raise PlanError(f"tensor {rec.name} row range {start}..{end} has byte range "
                                        f"{p.segment_byte_range}, expected {expect}")
                    ranges.append((start, end))
            covered = 0
            for start, end in sorted(ranges):
                if start != covered:
                    raise PlanError(f"tensor {rec.name} row coverage expected {covered}, got {start}")
                covered = end
            if covered != row_count:
                raise PlanError(f"tensor {rec.name} row coverage ends at {covered}, expected {row_count}")
        if self.policy == LAYER_SPLIT:
            previous = None
            for seg in index.segments:
                if seg.component_id not in selected or seg.kind != LAYER:
                    continue
                if seg.id not in layer_devices:
                    raise PlanError(f"layer segment {seg.id} has no assigned device")
                i = _device_index(self.devices, layer_devices[seg.id])
                if previous is not None and i < previous:
                    raise PlanError(f"layer segment {seg.id} backtracks to device {layer_devices[seg.id]!r}")
                previous = i
        for d in self.devices:
            used = self.used_bytes(d.id)
            if used > d.capacity:
                raise CapacityExceeded(d.id, used, d.capacity, "load plan placements")


def build_load_plan(index: PackageIndex, component_ids, devices, primary_device: str, policy: str) -> LoadPlan:
    """src/format/load_plan.rs:158-350"""
    devices = list(devices)
    primary = _validate_devices(devices, primary_device)
    component_ids = _selected_components(index, list(component_ids))
    selected = set(component_ids)
    remaining = [d.capacity for d in devices]
    placements = []

    def whole(rec, dev):
        return Placement(rec.component_id, rec.segment_id, rec.name, WHOLE,
                         (rec.segment_offset, rec.segment_offset + rec.byte_len), devices[dev].id)

    for rec in index.tensors:
        seg = index.segment(rec.segment_id)
        if rec.component_id not in selected or seg is None or seg.kind == LAYER:
            continue
        if rec.byte_len > remaining[primary]:
            raise CapacityExceeded(devices[primary].id, rec.byte_len, remaining[primary], f"tensor {rec.name}")
        placements.append(whole(rec, primary))
        remaining[primary] -= rec.byte_len

    layer_segments = sorted((s for s in index.segments if s.component_id in selected and s.kind == LAYER),
                            key=lambda s: (s.component_id, s.layer, s.id))
    cur = 0
    for seg in layer_segments:
        records = [r for r in index.tensors if r.segment_id == seg.id]
        if policy == LAYER_SPLIT:
            required = sum(r.byte_len for r in records)
            while cur < len(devices) and required > remaining[cur]:
                cur += 1
            if cur == len(devices):
                raise CapacityExceeded(devices[-1].id, required, remaining[-1], f"segment {seg.id}")
            placements.extend(whole(r, cur) for r in records)
            remaining[cur] -= required
        elif policy == TENSOR_SPLIT:
            for rec in records:
                row_count, row_bytes = row_layout(rec)
                row_start = 0
                while row_start < row_count:
                    while cur < len(devices) and remaining[cur] < row_bytes:
                        cur += 1
                    if cur == len(devices):
                        raise UnsplittableTensor(rec.name, row_bytes,
                                                 [(d.id, r) for d, r in zip(devices, remaining)],
                                                 "no remaining device can hold one complete row")
                    rows_here = min(remaining[cur] // row_bytes, row_count - row_start)
                    row_end = row_start + rows_here
                    placements.append(Placement(
                        rec.component_id, rec.segment_id, rec.name,
                        WHOLE if row_start == 0 and row_end == row_count else (row_start, row_end),
                        (rec.segment_offset + row_start * row_bytes, rec.segment_offset + row_end * row_bytes),
                        devices[cur].id))
                    remaining[cur] -= rows_here * row_bytes
                    row_start = row_end
        else:
            raise PlanError(f"unknown placement policy {policy!r}")
    plan = LoadPlan(component_ids, devices, primary_device, policy, placements)
    plan.validate(index)
    return plan


def balanced_devices(index: PackageIndex, world: int, prefix: str = "cuda", slack_rows: int = 0) -> list:
    """`world` logical devices in rank order whose capacities share the layer bytes equally (the primary, rank 0,
    also has room for the shared tensors).  TensorSplit fills devices greedily, so a package whose layer payload is
    one matrix (the column-sharded matmul) is cut into `world` equal row ranges when its rows divide by `world`;
    a whole model is cut at row granularity wherever a device fills up, and `slack_rows` adds that many of the
    largest rows to every device so the bytes lost at each cut do not overflow the last one."""
    shared = layers = max_row = 0
    for rec in index.tensors:
        if index.segment(rec.segment_id).kind == LAYER:
            layers += rec.byte_len
            max_row = max(max_row, row_layout(rec)[1])
        else:
            shared += rec.byte_len
    share = (layers + world - 1) // world + slack_rows * max_row
    return [LogicalDevice(f"{prefix}{r}", share + (shared if r == 0 else 0)) for r in range(world)]


def execute_plan(pkg, loader, plan: LoadPlan, index: PackageIndex, device_id: str, ctx=None) -> dict:
    """Upload this device's placements: {tensor name: [(row_start, row_end, QuantizedTensor)]} for the 2-D
    quantized tensors (one rmi_weight_upload_gguf per placement); other tensors (norm weights, rank one) come back
    as {name: [(row_start, row_end, uint8 view of the mapped bytes)]}.  `pkg` is the imported package, `loader` its
    GGUFLoader on the source file."""
    plan.validate(index)
    by_key = {(r.component_id, r.segment_id, r.name): r for r in index.tensors}
    out = {}
    for p in plan.placements:
        if p.device_id != device_id:
            continue
        rec = by_key[(p.component_id, p.segment_id, p.tensor_name)]
        row_count, row_bytes = row_layout(rec)
        start, end = (0, row_count) if p.slice is WHOLE else p.slice
        if len(rec.dims) == 2 and rec.ggml_type in (2, 8, 12, 14):
            item = pkg.QuantizedTensor.from_gguf(loader, rec.name, start, end, ctx=ctx)
        else:
            item = loader.tensor_slice(rec.name)[start * row_bytes:end * row_bytes]
        out.setdefault(rec.name, []).append((start, end, item))
    return out


def with_placements(plan: LoadPlan, placements) -> LoadPlan:
    return replace(plan, placements=list(placements))
