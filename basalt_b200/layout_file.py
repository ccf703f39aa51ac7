"""The model file's `experts` section and its `experts.layout` table: from bytes on disk to expert blobs resident in HBM.

The table is the reference's text format (Basalt: include/basalt/kernels/cpu/expert_layout.hpp:60-67, parsed by
src/kernels/cpu/expert_layout.cpp:133-203, written by tools/convert/model_sections.py:337-341 and described in
docs/model-file.md:230-241): a header `# experts vN: ... (n_expert E, total B)` and one line per layer,
`layer gu_type d_type offset blob_bytes` (from v7 also `up_type`).  A layer's E blobs `[gate | up | down | tail]` lie one
after another from `offset` inside the `experts` section.  Parsing is the library's (bsx_layout_parse); this module adds the
upload: a layer's blobs go through pinned staging buffers into one device tensor, and all-NVFP4 layers can be rewritten on
the way into the packed blocks the tensor-core kernels stream (bsx_expert_pack), so the raw blobs are never resident whole.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import capi
from .capi import ExpertLayout, LayoutInfo, LayoutRow

NEWEST_VERSION = 7          # kExpertLayoutVersion, expert_layout.hpp:67
READ_PAST_BYTES = 256       # zeroed bytes after a layer's last blob: rows are read 256 values at a time (docs/model-file.md:240-241)


@dataclass
class LayerRow:
    gu_type: int
    d_type: int
    up_type: int
    offset: int
    blob_bytes: int
    kernels: bool = True     # this library has kernels for the layer's formats


@dataclass
class ExpertTable:
    """basalt::kernels::cpu::ExpertLayout (expert_layout.hpp:17-35) for one model."""
    version: int
    n_layers: int
    n_expert: int
    n_embd: int
    n_ff: int
    swiglu_limit: float
    max_blob: int
    total: int
    rows: List[LayerRow] = field(default_factory=list)

    def blob_bytes(self, layer: int) -> int:
        return self.rows[layer].blob_bytes

    def layer_offset(self, layer: int) -> int:
        return self.rows[layer].offset

    def blob_offset(self, layer: int, expert: int) -> int:
        return self.layer_offset(layer) + expert * self.blob_bytes(layer)

    def layout(self, layer: int, gate_softcap: float = 0.0, up_softcap: float = 0.0) -> ExpertLayout:
        """The kernel-side geometry (bsx_expert_layout) of the layer's blobs."""
        r = self.rows[layer]
        L = ExpertLayout()
        capi.check("bsx_expert_layout_init", capi.lib().bsx_expert_layout_init(r.gu_type, r.d_type, r.up_type, self.n_embd, self.n_ff,
                                                                                self.swiglu_limit, gate_softcap, up_softcap, C.byref(L)))
        return L


def parse_layout_text(text: Union[str, bytes], n_layers: int, n_expert: int, n_embd: int, n_ff: int,
                      swiglu_limit: float = 0.0) -> ExpertTable:
    """expert_layout_load_text (expert_layout.cpp:133-203) without the process-wide table: returns the table, or raises
    ValueError with the reason where the reference returns false and fills `err`."""
    raw = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    if n_layers <= 0:
        raise ValueError("expert layout: no layers")
    rows = (LayoutRow * n_layers)()
    info = LayoutInfo()
    err = C.create_string_buffer(512)
    rc = capi.lib().bsx_layout_parse(raw, len(raw), n_layers, n_expert, n_embd, n_ff, swiglu_limit, rows, C.byref(info), err, len(err))
    if rc != 0:
        raise ValueError(err.value.decode("utf-8", "replace") or f"expert layout: error {rc}")
    return ExpertTable(version=info.version, n_layers=int(info.n_layers), n_expert=int(info.n_expert), n_embd=n_embd, n_ff=n_ff,
                       swiglu_limit=swiglu_limit, max_blob=int(info.max_blob), total=int(info.total),
                       rows=[LayerRow(r.gu_type, r.d_type, r.up_type, int(r.offset), int(r.blob_bytes), bool(r.kernels)) for r in rows])


def layout_text(layers: Sequence[Tuple[int, int, int]], n_expert: int, n_embd: int, n_ff: int, version: int = NEWEST_VERSION) -> str:
    """The text for layers given as (gu_type, d_type, up_type or -1), laid out contiguously from offset 0, in the form the
    reference's converter writes (model_sections.py:337-341); up to v6 the sixth column is left out."""
    lines, at = [], 0
    for l, (gt, dt, ut) in enumerate(layers):
        L = ExpertLayout()
        capi.check("bsx_expert_layout_init", capi.lib().bsx_expert_layout_init(gt, dt, ut, n_embd, n_ff, 0.0, 0.0, 0.0, C.byref(L)))
        cols = [l, gt, dt, at, int(L.bytes)] + ([L.up_type] if version >= 7 else [])
        lines.append(" ".join(str(c) for c in cols))
        at += int(L.bytes) * n_expert
    names = "layer gu_type d_type offset blob_bytes" + (" up_type" if version >= 7 else "")
    head = f"# experts v{version}: {names} (n_expert {n_expert}, total {at})"
    return head + "\n" + "\n".join(lines) + "\n"


class ExpertsSection:
    """The `experts` section of a model file (a path with the section's byte offset inside the file, or a uint8 buffer) read
    through its table.  The reference maps the section and pages experts in on demand (its VRAM / RAM tiers); on a B200 a
    layer's experts stay resident, so a layer is uploaded once, whole or as one rank's contiguous block of experts."""

    def __init__(self, source: Union[str, os.PathLike, bytes, bytearray, memoryview, np.ndarray], table: ExpertTable, base_offset: int = 0):
        self.table = table
        if isinstance(source, (str, os.PathLike)):
            size = os.path.getsize(source)
            if size < base_offset + table.total:
                raise ValueError(f"experts section: the file holds {size - base_offset} B after offset {base_offset}, the layout needs {table.total}")
            self.bytes = np.memmap(source, dtype=np.uint8, mode="r", offset=base_offset, shape=(table.total,))
        else:
            buf = np.frombuffer(source, dtype=np.uint8) if not isinstance(source, np.ndarray) else source.reshape(-1).view(np.uint8)
            if buf.size < base_offset + table.total:
                raise ValueError(f"experts section: {buf.size - base_offset} B given, the layout needs {table.total}")
            self.bytes = buf[base_offset:base_offset + table.total]

    def blob(self, layer: int, expert: int) -> np.ndarray:
        """One expert's blob as a host view (no copy)."""
        t = self.table
        if not (0 <= layer < t.n_layers and 0 <= expert < t.n_expert):
            raise IndexError("layer or expert out of range")
        o = t.blob_offset(layer, expert)
        return self.bytes[o:o + t.blob_bytes(layer)]

    def load_layer(self, layer: int, device, experts: Optional[range] = None, pack: bool = False, chunk_experts: int = 32,
                   stream=None) -> Tuple[torch.Tensor, ExpertLayout]:
        """Uploads experts `experts` (default: all; a contiguous range, e.g. one rank's block) of `layer`.

        Returns (blobs [n][stride] uint8 on `device`, layout).  pack=False: raw ggml blobs, stride = blob bytes rounded up to
        16, followed by READ_PAST_BYTES zero bytes.  pack=True (all-NVFP4 layers): the packed blocks of bsx_expert_pack; raw
        bytes pass through a device staging area of chunk_experts blobs only.  Host reads go through two pinned buffers so
        the copy of one chunk overlaps the page-in of the next."""
        from . import moe
        t = self.table
        L = t.layout(layer)
        experts = range(t.n_expert) if experts is None else experts
        if experts.step != 1 or experts.start < 0 or experts.stop > t.n_expert:
            raise ValueError("experts must be a contiguous range inside the layer")
        n, blob = len(experts), t.blob_bytes(layer)
        dev = torch.device(device)
        stride = (blob + 15) // 16 * 16
        st = torch.cuda.current_stream(dev) if stream is None else stream
        if pack:
            nb = int(capi.lib().bsx_expert_packed_bytes(C.byref(L)))
            if not nb:
                raise ValueError("layer not covered by the packed path (all-NVFP4, n_embd % 256 == 0, n_ff % 256 == 0)")
            out = torch.empty((n, nb), dtype=torch.uint8, device=dev)
            stage = torch.zeros((min(chunk_experts, max(n, 1)), stride), dtype=torch.uint8, device=dev)
        else:
            flat = torch.zeros(n * stride + READ_PAST_BYTES, dtype=torch.uint8, device=dev)
            out = flat[:n * stride].view(n, stride)
            stage = None
        c = max(1, min(chunk_experts, n))
        pinned = [torch.empty((c, blob), dtype=torch.uint8).pin_memory() for _ in range(2)]
        free = [torch.cuda.Event() for _ in range(2)]
        with torch.cuda.stream(st):
            for i, e0 in enumerate(range(0, n, c)):
                m = min(c, n - e0)
                o = t.blob_offset(layer, experts.start + e0)
                buf = pinned[i & 1]
                if i >= 2:
                    free[i & 1].synchronize()       # the copy that last read this buffer has finished
                buf[:m].numpy()[...] = self.bytes[o:o + m * blob].reshape(m, blob)
                dst = stage[:m] if pack else out[e0:e0 + m]
                dst[:, :blob].copy_(buf[:m], non_blocking=True)
                free[i & 1].record(st)
                if pack:
                    for j in range(m):
                        capi.check("bsx_expert_pack", capi.lib().bsx_expert_pack(C.byref(L), stage[j].data_ptr(), out[e0 + j].data_ptr(),
                                                                                  moe._stream(st)))
        st.synchronize()
        return out, L
