"""Token-stream readers: flat uint16 `.bin` files -> (x, y) int64 batches of shape [B, S].

Sampling contract (behaviour parity with reference src/data/utils.py:411-696 so that a
run on the same file with the same seed sees the same batches):

* without replacement: per epoch e, `rng = default_rng(seed + e)`; `order = rng.permutation(
  (n - S - 1) // S - 1)`; `offset = rng.integers(S)`; global batch j covers
  `order[j*B:(j+1)*B] * S + offset`; rank r of N reads global batches r, N+r, 2N+r, ...;
  the epoch rolls over after `len(order) // B` global batches.
* with replacement: `default_rng(seed + step*N + rank).integers(n - S - 1, size=B)`.
* no collectives anywhere: every rank derives its indices locally.

The gather is a single vectorised fancy-index into the stream (the reference stacks one
slice per sequence), and a batch can be written straight into caller-provided pinned
buffers (`sample_batch(out=(x_pinned, y_pinned))`) so that the host-to-device copy that
follows is asynchronous.
"""
from __future__ import annotations

import queue
import threading
import time
from pathlib import Path
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


_DP_LAYOUT = None      # (data-parallel size, this process's data-parallel rank) when it differs from the process group's


def set_data_parallel_layout(size: int, rank: int):
    """Tensor parallelism: the ranks of one tp group must read the same batches, so readers shard the data over the
    data-parallel replicas instead of over all processes.  `None, None` restores the default."""
    global _DP_LAYOUT
    _DP_LAYOUT = None if size is None else (int(size), int(rank))


def _dist_info(auto_shard: bool):
    if auto_shard and _DP_LAYOUT is not None:
        return _DP_LAYOUT
    if auto_shard and dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class DataReader:
    def __init__(self, data_src, local_batch_size, sequence_length, seed=1337,
                 with_replacement=False, auto_shard=True, keep_in_ram=False,
                 world_size: Optional[int] = None, rank: Optional[int] = None):
        if isinstance(data_src, (str, Path)):
            self.data_path = Path(data_src)
            self.keep_in_ram = keep_in_ram
            self.data = np.array(np.memmap(self.data_path, dtype=np.uint16, mode="r")) if keep_in_ram else None
        elif isinstance(data_src, (np.ndarray, np.memmap)):
            self.data_path = None
            self.data = data_src
            self.keep_in_ram = True
        else:
            raise TypeError(f"unsupported data source {type(data_src)}")
        self.local_batch_size = local_batch_size
        self.sequence_length = sequence_length
        self.seed = seed
        self.with_replacement = with_replacement
        self.num_tokens = len(self._get_data())
        if world_size is not None:
            self.world_size, self.rank = world_size, (rank or 0)
        else:
            self.world_size, self.rank = _dist_info(auto_shard)
        self.last_epoch = None
        self.order = None
        self.epoch_offset = None
        self.step = 0
        self.total_possible_local_batches = 0
        self.num_batches_of_seqlen = 0
        self._arange = np.arange(sequence_length + 1, dtype=np.int64)
        if with_replacement:
            n_seq = len(self) // sequence_length - 1
            self.num_batches_of_seqlen = (n_seq // local_batch_size) // self.world_size
        else:
            self._shuffle_epoch(0)

    # ---- storage -------------------------------------------------------------------------
    def _get_data(self):
        if self.data is not None:
            return self.data
        # re-open per access: a long-lived memmap grows the resident set as pages are touched
        return np.memmap(self.data_path, dtype=np.uint16, mode="r")

    def __len__(self):
        return self.num_tokens - self.sequence_length - 1

    def __getitem__(self, idx):
        assert 0 <= idx < len(self)
        w = self._get_data()[idx: idx + self.sequence_length + 1].astype(np.int64)
        return torch.from_numpy(w[:-1].copy()), torch.from_numpy(w[1:].copy())

    # ---- index plan ------------------------------------------------------------------------
    def _shuffle_epoch(self, epoch: int):
        rng = np.random.default_rng(self.seed + epoch)
        self.order = rng.permutation(len(self) // self.sequence_length - 1)
        self.epoch_offset = rng.integers(self.sequence_length)
        self.last_epoch = epoch
        self.total_possible_local_batches = len(self.order) // self.local_batch_size
        self.num_batches_of_seqlen = self.total_possible_local_batches // self.world_size

    def _indices(self, step: int, peek: bool = False) -> np.ndarray:
        if self.with_replacement:
            rng = np.random.default_rng(self.seed + step * self.world_size + self.rank)
            return rng.integers(len(self), size=self.local_batch_size)
        j = self.world_size * step + self.rank
        per_epoch = self.total_possible_local_batches
        epoch, k = divmod(j, per_epoch)
        if epoch != self.last_epoch:
            if peek:
                rng = np.random.default_rng(self.seed + epoch)
                order = rng.permutation(len(self) // self.sequence_length - 1)
                off = rng.integers(self.sequence_length)
                return order[k * self.local_batch_size:(k + 1) * self.local_batch_size] * self.sequence_length + off
            print(f"Shuffling. Rank {self.rank}. File: {self.data_path}. Epoch: {epoch}.")
            self._shuffle_epoch(epoch)
        sl = self.order[k * self.local_batch_size:(k + 1) * self.local_batch_size]
        return sl * self.sequence_length + self.epoch_offset

    def set_step(self, step: int):
        self.step = step

    def sample_batch(self, out=None):
        data = self._get_data()
        starts = np.asarray(self._indices(self.step), dtype=np.int64)
        self.step += 1
        win = data[starts[:, None] + self._arange[None, :]]
        if out is not None:
            x_out, y_out = out
            x_out.numpy()[...] = win[:, :-1]
            y_out.numpy()[...] = win[:, 1:]
            return x_out, y_out
        win = win.astype(np.int64)
        return (torch.from_numpy(np.ascontiguousarray(win[:, :-1])),
                torch.from_numpy(np.ascontiguousarray(win[:, 1:])))

    def preview_next_samples(self, num_preview=3):
        """Start indices of the next batches without advancing (used to check a resume)."""
        return [self._indices(self.step + i, peek=True)[:5].tolist() for i in range(num_preview)]

    # ---- bookkeeping -------------------------------------------------------------------------
    def num_batches(self):
        if self.with_replacement:
            return self.num_tokens // self.local_batch_size
        return self.num_batches_of_seqlen

    def num_batches_for_switching(self):
        return self.num_batches_of_seqlen

    def state_dict(self):
        st = {"step": self.step}
        if not self.with_replacement:
            st.update(last_epoch=self.last_epoch or 0,
                      order=None if self.order is None else self.order.copy(),
                      epoch_offset=self.epoch_offset or 0,
                      total_possible_local_batches=self.total_possible_local_batches,
                      num_batches_of_seqlen=self.num_batches_of_seqlen)
        return st

    def load_state_dict(self, st):
        self.step = st.get("step", 0)
        if self.with_replacement:
            return
        if st.get("order") is not None:
            self.last_epoch = st.get("last_epoch", 0)
            self.order = np.asarray(st["order"])
            self.epoch_offset = st.get("epoch_offset", 0)
            self.total_possible_local_batches = st.get("total_possible_local_batches", 0)
            self.num_batches_of_seqlen = st.get("num_batches_of_seqlen", 0)
        else:
            per_epoch = max(1, self.total_possible_local_batches)
            self._shuffle_epoch((self.world_size * self.step + self.rank) // per_epoch)


class AsyncFileLoader:
    """Background thread that reads the next token file into RAM while training runs."""

    def __init__(self):
        self._requests: "queue.Queue" = queue.Queue()
        self._results: "queue.Queue" = queue.Queue()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="adana-file-loader")
        self._thread.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                path = self._requests.get(timeout=0.2)
            except queue.Empty:
                continue
            if path is None:
                break
            try:
                t0 = time.time()
                arr = np.array(np.memmap(path, dtype=np.uint16, mode="r"))
                self._results.put((path, arr, time.time() - t0))
            except Exception as e:  # surfaced to the consumer as a miss
                self._results.put((path, None, repr(e)))

    def start_loading(self, path):
        self._requests.put(Path(path))

    def get_loaded_file(self, path=None, timeout=5.0):
        try:
            p, arr, _ = self._results.get(timeout=timeout)
        except queue.Empty:
            return None
        if arr is None or (path is not None and Path(path) != p):
            return None
        return p, arr

    def clear_queue(self):
        for q in (self._requests, self._results):
            while True:
                try:
                    q.get_nowait()
                except queue.Empty:
                    break

    def shutdown(self):
        self._stop.set()
        self._requests.put(None)


class MultiFileDataReader:
    """Cycles over `train_XXXX.bin` files: current file in RAM, next one pre-loaded by a thread.

    File k is sampled with seed `seed + 1000*k`; a rank moves on when it has drawn its share
    of the current file (decided locally, no collectives).  Parity: reference
    src/data/utils.py:123-409.
    """

    def __init__(self, data_files, local_batch_size, sequence_length, seed=1337,
                 with_replacement=False, auto_shard=True, keep_in_ram=False):
        if isinstance(data_files, (str, Path)):
            self.file_paths, self.is_single_file = [Path(data_files)], True
        elif isinstance(data_files, dict):
            files = sorted(Path(v) for k, v in data_files.items() if k.startswith("train_"))
            if not files:
                raise ValueError("No train files found in data_files dict")
            self.file_paths, self.is_single_file = files, False
        elif isinstance(data_files, (list, tuple)):
            self.file_paths, self.is_single_file = [Path(f) for f in data_files], False
        else:
            raise ValueError(f"Unsupported data_files type: {type(data_files)}")
        self.local_batch_size = local_batch_size
        self.sequence_length = sequence_length
        self.seed = seed
        self.with_replacement = with_replacement
        self.auto_shard = auto_shard
        self.world_size, self.rank = _dist_info(auto_shard)
        self.current_file_idx = 0
        self.async_loader = AsyncFileLoader()
        self.disable_coordination = False
        self._open(0, None)
        self.num_tokens = len(self.current_data) * len(self.file_paths)
        self.step = 0

    def _open(self, idx: int, preloaded):
        self.current_file_idx = idx
        path = self.file_paths[idx]
        self.current_data = preloaded if preloaded is not None else np.array(
            np.memmap(path, dtype=np.uint16, mode="r"))
        self.current_reader = DataReader(self.current_data, self.local_batch_size,
                                         self.sequence_length, seed=self.seed + 1000 * idx,
                                         with_replacement=self.with_replacement,
                                         auto_shard=self.auto_shard, keep_in_ram=True)
        if len(self.file_paths) > 1:
            self.async_loader.start_loading(self.file_paths[(idx + 1) % len(self.file_paths)])

    def _advance_file(self):
        nxt = (self.current_file_idx + 1) % len(self.file_paths)
        got = self.async_loader.get_loaded_file(self.file_paths[nxt], timeout=5.0)
        self._open(nxt, None if got is None else got[1])

    def __len__(self):
        return len(self.current_reader) * len(self.file_paths)

    def __getitem__(self, idx):
        return self.current_reader[idx % len(self.current_reader)]

    def set_step(self, step):
        self.step = step
        self.current_reader.set_step(step)

    def sample_batch(self, out=None):
        if not self.is_single_file and self.step >= self.current_file_num_batches():
            self._advance_file()
            self.step = 0
        self.step += 1
        return self.current_reader.sample_batch(out=out)

    def num_batches(self):
        return self.current_reader.num_batches() * len(self.file_paths)

    def current_file_num_batches(self):
        return self.current_reader.num_batches_for_switching()

    def state_dict(self):
        return {"current_file_idx": self.current_file_idx, "step": self.step,
                "current_reader_state": self.current_reader.state_dict()}

    def load_state_dict(self, st):
        self.async_loader.clear_queue()
        self._open(st.get("current_file_idx", 0), None)
        self.step = st.get("step", 0)
        if "current_reader_state" in st:
            self.current_reader.load_state_dict(st["current_reader_state"])
        else:
            self.current_reader.set_step(self.step)

    def __del__(self):
        loader = getattr(self, "async_loader", None)
        if loader is not None:
            loader.shutdown()


class PinnedBatchStager:
    """Double-buffered pinned host staging + asynchronous host-to-device copies of batches.

    `next_batch()` returns device tensors for batch i while batch i+1 is being gathered into
    the other pinned buffer; the copy runs on a side stream and the consumer stream waits on
    an event, so input transfer overlaps compute.  (The reference pins and copies inline:
    src/optim/utils.py:74-83.)
    """

    def __init__(self, reader, device, depth: int = 2, lookahead: bool = True):
        # lookahead=False stages each batch when it is asked for, so that the reader's step
        # always equals the number of consumed batches (exact checkpoint/resume positions).
        self.lookahead = lookahead
        self.reader = reader
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        B, S = reader.local_batch_size, reader.sequence_length
        self.depth = depth
        self._host = [(torch.empty((B, S), dtype=torch.int64, pin_memory=self.cuda),
                       torch.empty((B, S), dtype=torch.int64, pin_memory=self.cuda)) for _ in range(depth)]
        self._dev = [(torch.empty((B, S), dtype=torch.int64, device=self.device),
                      torch.empty((B, S), dtype=torch.int64, device=self.device)) for _ in range(depth)] if self.cuda else None
        self._events = [torch.cuda.Event() for _ in range(depth)] if self.cuda else None
        self._stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._slot = 0
        self._primed = False
        self.bytes_per_batch = 2 * B * S * 8

    def _stage(self, slot):
        if self.cuda:
            self._events[slot].synchronize()  # the last copy out of this pinned slot is done
        x, y = self.reader.sample_batch(out=self._host[slot])
        if not self.cuda:
            return
        # The kernels that still read this device slot were queued on the consumer's stream before this call, so the
        # copy stream waits for everything queued there so far.  (The stream is looked up OUTSIDE the `with` block:
        # inside it the current stream is the copy stream itself and the wait would order nothing.)
        consumer = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self._stream):
            self._stream.wait_stream(consumer)
            self._dev[slot][0].copy_(x, non_blocking=True)
            self._dev[slot][1].copy_(y, non_blocking=True)
            self._events[slot].record(self._stream)

    def next_batch(self):
        if not self.lookahead:
            slot = self._slot
            self._stage(slot)
            self._slot = (slot + 1) % self.depth
            if self.cuda:
                torch.cuda.current_stream(self.device).wait_event(self._events[slot])
                return self._dev[slot]
            return self._host[slot][0].clone(), self._host[slot][1].clone()
        if not self._primed:
            self._stage(self._slot)
            self._primed = True
        slot = self._slot
        nxt = (slot + 1) % self.depth
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self._events[slot])
            out = self._dev[slot]
        else:
            out = (self._host[slot][0].clone(), self._host[slot][1].clone())
        self._stage(nxt)
        self._slot = nxt
        return out
