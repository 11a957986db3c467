"""Datasets, loader, transforms (crates/incin-data: loader.rs:9-120, transforms/mod.rs:13-211,
vision/mnist.rs, hub.rs).  The loader keeps the reference's shape — shuffle, worker threads feeding a bounded
queue of ``2 * workers + 2`` batches, a collate function — and adds what a GPU step needs: batches are
collated into PINNED host memory and copied to the device asynchronously one batch ahead of the consumer.
"""
from __future__ import annotations

import gzip
import os
import queue
import struct
import threading
from pathlib import Path
from typing import Callable, Sequence

import torch


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, i: int):
        raise NotImplementedError


class TensorDataset(Dataset):
    def __init__(self, *tensors: torch.Tensor):
        if not tensors or any(t.shape[0] != tensors[0].shape[0] for t in tensors):
            raise ValueError("tensors must share their first dimension")
        self.tensors = tensors

    def __len__(self):
        return self.tensors[0].shape[0]

    def __getitem__(self, i):
        return tuple(t[i] for t in self.tensors)


class SyntheticTokens(Dataset):
    """Uniform random token ids of a fixed shape (what the benchmarks train on: no dataset on the box)."""

    def __init__(self, n: int, seq_len: int, vocab: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randint(0, vocab, (n, seq_len + 1), generator=g)

    def __len__(self):
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i, :-1], self.x[i, 1:]


def default_collate(samples: Sequence):
    first = samples[0]
    if isinstance(first, (tuple, list)):
        return tuple(default_collate([s[k] for s in samples]) for k in range(len(first)))
    if isinstance(first, torch.Tensor):
        return torch.stack(list(samples))
    return torch.as_tensor(list(samples))


def _pin(batch):
    if isinstance(batch, tuple):
        return tuple(_pin(b) for b in batch)
    return batch.pin_memory() if torch.cuda.is_available() and isinstance(batch, torch.Tensor) else batch


def _to(batch, device):
    if isinstance(batch, tuple):
        return tuple(_to(b, device) for b in batch)
    return batch.to(device, non_blocking=True) if isinstance(batch, torch.Tensor) else batch


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 1, shuffle: bool = False, workers: int = 0,
                 collate: Callable = default_collate, drop_last: bool = False, seed: int = 0, device=None,
                 pin_memory: bool | None = None, native: bool = False):
        if batch_size < 1:
            raise ValueError("batch_size must be >= 1")
        self.dataset, self.batch_size, self.shuffle, self.workers = dataset, batch_size, shuffle, workers
        self.collate, self.drop_last, self.seed, self.epoch = collate, drop_last, seed, 0
        self.device = torch.device(device) if device is not None else None
        self.pin = (self.device is not None and self.device.type == "cuda") if pin_memory is None else pin_memory
        # native=True: batches of a TensorDataset are gathered by the C++ loader (csrc/runtime/loader.cpp: worker
        # threads, ordered delivery, bounded ring) instead of Python threads.  Its permutation is its own (splitmix64
        # Fisher-Yates of seed + epoch), so the batch sequence differs from the Python path for the same seed.
        self.native = bool(native) and isinstance(dataset, TensorDataset) and collate is default_collate \
            and 1 <= len(dataset.tensors) <= 2 and all(t.device.type == "cpu" for t in dataset.tensors)
        self._native_loader = None

    def __len__(self):
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def _batches(self):
        n = len(self.dataset)
        order = torch.randperm(n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist() \
            if self.shuffle else list(range(n))
        for i in range(0, n, self.batch_size):
            idx = order[i:i + self.batch_size]
            if len(idx) < self.batch_size and self.drop_last:
                return
            yield idx

    def _load(self, idx):
        b = self.collate([self.dataset[i] for i in idx])
        return _pin(b) if self.pin else b

    def _native_iter(self):
        from ..runtime import NativeBatchLoader
        if self._native_loader is None:
            ts = self.dataset.tensors
            self._native_loader = NativeBatchLoader(ts[0], ts[1] if len(ts) == 2 else None, batch_size=self.batch_size,
                                                    shuffle=self.shuffle, drop_last=self.drop_last, seed=self.seed,
                                                    workers=max(self.workers, 1), prefetch=4, pin=False)
        self._native_loader.epoch = self.epoch
        for b in self._native_loader:
            b = b if isinstance(b, tuple) else (b,)     # fresh tensors per batch (the loader is not in pinned-ring mode)
            yield _pin(b) if self.pin else b

    def _host_iter(self):
        if self.native:
            yield from self._native_iter()
            return
        if self.workers <= 0:
            for idx in self._batches():
                yield self._load(idx)
            return
        work: queue.Queue = queue.Queue()
        done: queue.Queue = queue.Queue(maxsize=2 * self.workers + 2)   # bounded: workers stall, memory does not grow
        batches = list(self._batches())
        for k, idx in enumerate(batches):
            work.put((k, idx))

        def worker():
            while True:
                try:
                    k, idx = work.get_nowait()
                except queue.Empty:
                    return
                try:
                    done.put((k, self._load(idx)))
                except Exception as e:   # surface loader errors in the consumer thread
                    done.put((k, e))
        threads = [threading.Thread(target=worker, daemon=True) for _ in range(self.workers)]
        for t in threads:
            t.start()
        pending, nxt = {}, 0
        while nxt < len(batches):     # deliver in order regardless of which worker finished first
            while nxt not in pending:
                k, b = done.get()
                pending[k] = b
            b = pending.pop(nxt)
            if isinstance(b, Exception):
                raise b
            yield b
            nxt += 1

    def __iter__(self):
        it = self._host_iter()
        self.epoch += 1
        if self.device is None:
            yield from it
            return
        prev = None
        for b in it:                   # one batch ahead: H2D copy of batch i+1 overlaps the step on batch i
            cur = _to(b, self.device)
            if prev is not None:
                yield prev
            prev = cur
        if prev is not None:
            yield prev


# ------------------------------------------------------------------------------------------------ transforms
class Compose:
    def __init__(self, *ts):
        self.ts = ts

    def __call__(self, x):
        for t in self.ts:
            x = t(x)
        return x


class Normalize:
    def __init__(self, mean, std):
        self.mean, self.std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)
        if (self.std == 0).any():
            raise ValueError("std must be non-zero")

    def __call__(self, x):
        shape = (-1,) + (1,) * (x.dim() - 1)
        return (x - self.mean.reshape(shape)) / self.std.reshape(shape)


class Scale:
    def __init__(self, factor: float):
        self.factor = factor

    def __call__(self, x):
        return x * self.factor


class RandomHorizontalFlip:
    def __init__(self, p: float = 0.5, seed: int = 0):
        self.p, self.g = p, torch.Generator().manual_seed(seed)

    def __call__(self, x):
        return x.flip(-1) if torch.rand((), generator=self.g).item() < self.p else x


class CenterCrop:
    def __init__(self, h: int, w: int):
        self.h, self.w = h, w

    def __call__(self, x):
        H, W = x.shape[-2:]
        if self.h > H or self.w > W:
            raise ValueError(f"crop {self.h}x{self.w} larger than image {H}x{W}")
        t, l = (H - self.h) // 2, (W - self.w) // 2
        return x[..., t:t + self.h, l:l + self.w]


# ------------------------------------------------------------------------------------------------ MNIST / hub
def _read_idx(path: Path) -> torch.Tensor:
    raw = gzip.open(path, "rb").read() if path.suffix == ".gz" else path.read_bytes()
    zero, dtype, nd = struct.unpack_from(">HBB", raw, 0)
    if zero != 0 or dtype != 0x08:
        raise ValueError(f"{path}: not an unsigned-byte IDX file")
    dims = struct.unpack_from(f">{nd}I", raw, 4)
    data = torch.frombuffer(bytearray(raw[4 + 4 * nd:]), dtype=torch.uint8)
    return data.reshape(dims)


class MnistDataset(Dataset):
    """Reads the IDX files from ``root`` (``train-images-idx3-ubyte[.gz]`` ...).  There is no network here, so
    nothing is downloaded: a missing file raises with the path that was expected."""

    def __init__(self, root, train: bool = True, transform: Callable | None = None):
        root, stem = Path(root), ("train" if train else "t10k")
        def find(name):
            for p in (root / name, root / (name + ".gz")):
                if p.exists():
                    return p
            raise FileNotFoundError(f"{root / name}[.gz] not found (offline build: place the MNIST IDX files there)")
        self.images = _read_idx(find(f"{stem}-images-idx3-ubyte")).float().div_(255.0).unsqueeze(1)
        self.labels = _read_idx(find(f"{stem}-labels-idx1-ubyte")).long()
        self.transform = transform

    def __len__(self):
        return self.labels.shape[0]

    def __getitem__(self, i):
        x = self.images[i]
        return (self.transform(x) if self.transform else x), self.labels[i]


class HubApi:
    """Model-hub cache lookup (``INCIN_HUB_CACHE_DIR`` / ``INCIN_HUB_TOKEN``).  Offline: only files already in the
    cache resolve; anything else raises instead of attempting a download."""

    def __init__(self, cache_dir=None):
        self.cache = Path(cache_dir or os.environ.get("INCIN_HUB_CACHE_DIR", os.path.expanduser("~/.cache/incin/hub")))

    def path(self, repo: str, filename: str) -> Path:
        p = self.cache / repo.replace("/", "--") / filename
        if not p.exists():
            raise FileNotFoundError(f"{repo}/{filename} is not in the hub cache {self.cache} and this build has no network")
        return p

    def from_pretrained(self, repo: str, filename: str = "model.safetensors"):
        from ..io import load_safetensors
        return load_safetensors(self.path(repo, filename))


class Collate:
    """A batch-assembly policy as an object (crates/incin-data/src/loader.rs ``Collate``): ``Collate()`` stacks samples
    field by field like :func:`default_collate`; ``Collate(pad_value=0)`` first pads variable-length leading axes of each
    field to the longest sample of the batch (token sequences), and ``Collate(fn)`` wraps any function."""

    def __init__(self, fn: Callable | None = None, pad_value=None):
        self.fn, self.pad_value = fn, pad_value

    def __call__(self, samples: Sequence):
        if self.fn is not None:
            return self.fn(samples)
        if self.pad_value is None:
            return default_collate(samples)
        first = samples[0]
        fields = list(zip(*samples)) if isinstance(first, (tuple, list)) else [samples]
        out = []
        for col in fields:
            col = [torch.as_tensor(c) for c in col]
            if col[0].dim() == 0 or len({c.shape[0] for c in col}) == 1:
                out.append(torch.stack(col))
                continue
            n = max(c.shape[0] for c in col)
            padded = [torch.cat([c, c.new_full((n - c.shape[0],) + tuple(c.shape[1:]), self.pad_value)]) for c in col]
            out.append(torch.stack(padded))
        return tuple(out) if isinstance(first, (tuple, list)) else out[0]


def from_pretrained(repo: str, filename: str = "model.safetensors", cache_dir=None):
    """Tensors of a cached hub checkpoint (``HubApi(cache_dir).from_pretrained``)."""
    return HubApi(cache_dir).from_pretrained(repo, filename)
