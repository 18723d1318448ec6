"""Binding a checkpoint's tensors to a model's parameters by name.

The rules follow the reference's loader
(crates/esp/src/infer/decoder/loader.rs:277-308, :425-462, :490-570): every
tensor the configuration calls for must be present with its exact shape, and a
checkpoint that carries a tensor nothing reads is refused (its weights would
compute something this decoder does not), except names that are known to be
derivable from the configuration.  All problems are gathered into one error.
"""
from __future__ import annotations

import torch

from ..errors import InvalidWeights
from .safetensors_io import open_model_folder, read_tensor

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


class FolderSource:
    """Tensors of a model folder (model.safetensors or its shards).

    A destination on the GPU is filled straight from the file: the tensor's bytes are read in chunks into
    two pinned buffers in turn and copied to the device asynchronously, so that reading the next chunk
    overlaps the copy of this one and no tensor passes through pageable memory; whether the values are finite is
    checked on the device, one status word per tensor, and reported once at the end (``finish``) with the
    tensors' names.  A checkpoint of a hundred gigabytes then loads at the speed of the disk."""

    CHUNK_BYTES = 64 << 20

    def __init__(self, folder):
        self.metas = open_model_folder(folder)
        self._pinned = None          # two pinned byte buffers
        self._landed = [None, None]  # the event after the last copy out of each
        self._turn = 0
        self._flags = None           # int32 [tensors]: non-zero where a tensor holds a non-finite value
        self._flag_names = []

    def names(self):
        return list(self.metas)

    def dtype(self, name):
        return self.metas[name].dtype

    def shape(self, name):
        return tuple(self.metas[name].shape)

    def read_into(self, name, view: torch.Tensor) -> None:
        meta = self.metas[name]
        if view.is_cuda and meta.dtype in (torch.float32, torch.bfloat16):
            self._stream_to_device(meta, view)
            return
        t = read_tensor(meta)
        # non-finite weights are refused (crates/esp/src/infer/decoder/weight_format.rs:129-131)
        if not bool(torch.isfinite(t if t.dtype == torch.float32 else t.float()).all()):
            raise InvalidWeights(f"{name} holds values that are not finite")
        view.copy_(t.to(view.dtype) if t.dtype != view.dtype else t, non_blocking=False)

    def _stream_to_device(self, meta, view: torch.Tensor) -> None:
        from ..csrc import ops
        device = view.device
        n_bytes = meta.hi - meta.lo
        direct = view.is_contiguous() and view.dtype == meta.dtype
        # the file's bytes land in the destination itself, or (another dtype, or a strided destination) in a
        # device tensor of the stored dtype that is then converted into it
        target = view if direct else torch.empty(meta.shape, dtype=meta.dtype, device=device)
        flat = target.view(-1).view(torch.uint8)
        if self._pinned is None:
            self._pinned = [torch.empty(self.CHUNK_BYTES, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        if self._flags is None or len(self._flag_names) >= self._flags.numel():
            self._collect()
            self._flags = torch.zeros(4096, dtype=torch.int32, device=device)
        with open(meta.file, "rb", buffering=0) as f:
            f.seek(meta.lo)
            done = 0
            while done < n_bytes:
                n = min(self.CHUNK_BYTES, n_bytes - done)
                b = self._turn % 2
                self._turn += 1
                if self._landed[b] is not None:
                    self._landed[b].synchronize()             # the last copy out of this buffer is done
                got = f.readinto(memoryview(self._pinned[b].numpy())[:n])
                if got != n:
                    raise InvalidWeights(f"{meta.file.name}: {meta.name} ends early ({done + (got or 0)} of {n_bytes} bytes)")
                flat[done:done + n].copy_(self._pinned[b][:n], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                self._landed[b] = ev
                done += n
        # non-finite weights are refused (crates/esp/src/infer/decoder/weight_format.rs:129-131): checked on the
        # device, told at the end
        i = len(self._flag_names)
        self._flag_names.append(meta.name)
        if n_bytes:
            ops.finite_check(target.view(-1), self._flags[i:i + 1], bit=1)
        if not direct:
            view.copy_(target)

    def _collect(self) -> None:
        if self._flags is not None and self._flag_names:
            bad = [n for n, f in zip(self._flag_names, self._flags[:len(self._flag_names)].tolist()) if f]
            self._flag_names = []
            self._flags.zero_()
            if bad:
                shown = ", ".join(bad[:8]) + (" ..." if len(bad) > 8 else "")
                raise InvalidWeights(f"{shown} hold{'s' if len(bad) == 1 else ''} values that are not finite")

    def finish(self) -> None:
        """Waits for the copies and raises InvalidWeights naming every tensor with a non-finite value."""
        self._collect()
        self._pinned = None
        self._landed = [None, None]


def check_names_and_shapes(specs: list, source, tolerated_suffixes=()) -> None:
    """One InvalidWeights that lists missing and unexpected tensors, wrong
    shapes and wrong dtypes; nothing if all is well."""
    wanted = {}
    for s in specs:
        if s.name in wanted and wanted[s.name].shape != s.shape:
            raise InvalidWeights(f"two parts declare {s.name} with different shapes")
        wanted[s.name] = s
    have = set(source.names())
    missing = sorted(n for n, s in wanted.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in wanted and not any(n.endswith(t) for t in tolerated_suffixes))
    wrong_shape, wrong_dtype = [], []
    for n in sorted(have & set(wanted)):
        if tuple(source.shape(n)) != tuple(wanted[n].shape):
            wrong_shape.append(f"{n}: stored {list(source.shape(n))}, expected {list(wanted[n].shape)}")
        if source.dtype(n) not in _FLOAT_DTYPES:
            wrong_dtype.append(f"{n}: stored as {source.dtype(n)}")
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = ["the checkpoint does not match the configuration:"]

    def add(title, items):
        if items:
            shown = items[:12]
            lines.append(f"  {title} ({len(items)}): " + "; ".join(shown) + (" ..." if len(items) > len(shown) else ""))

    add("missing tensors", missing)
    add("unexpected tensors (nothing in this configuration reads them)", unexpected)
    add("wrong shapes", wrong_shape)
    add("dtypes that are not floating point", wrong_dtype)
    raise InvalidWeights("\n".join(lines))


def load_into(root, source, rt, tolerated_suffixes=None) -> None:
    """Checks the source against the parameters of ``root`` (a model, or any
    part with its children), lets every part allocate its storage and fills it."""
    from ..parts import walk
    parts = list(walk(root))
    specs = [s for part in parts for s in part.param_specs()]
    if tolerated_suffixes is None:
        tolerated_suffixes = getattr(getattr(root, "plan", None), "tolerated_suffixes", ())
    check_names_and_shapes(specs, source, tolerated_suffixes)
    have = set(source.names())
    stored = {s.name: source.dtype(s.name) for s in specs if s.name in have}
    views = {}
    for part in parts:
        views.update(part.allocate(stored, rt))
    for name, view in views.items():
        if name not in have:
            raise InvalidWeights(f"a part asked for {name}, which the checkpoint lacks")
        source.read_into(name, view)
    if hasattr(source, "finish"):
        source.finish()
    for part in parts:
        part.finalize()
