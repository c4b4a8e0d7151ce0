"""Micro-batch input pipeline.

Constructor signature, attributes and the batch dictionary follow ``picotron/data.py:12-137`` of the
reference: samples are ``seq_length + 1`` token windows, the sampler shards them over **data-parallel**
ranks only (every TP/PP/CP rank of one DP replica sees the same samples), the collate step slices this
rank's **context-parallel** chunk and builds the shifted targets and position ids, and iteration is
infinite (the epoch counter is bumped on exhaustion).

Two sources:

* ``dataset_name == "synthetic"`` -- uniform-random token ids from a fixed seed, generated on the fly
  (sample ``i`` depends only on ``(seed, i)``, so every rank of a replica draws the same window without
  communication). This is what benchmarks and tests use; it needs no network.
* anything else -- a HF ``datasets`` dataset tokenised with the model's tokenizer and grouped into
  windows, exactly like the reference (tokenizer built on rank 0 and broadcast). A ``dataset_name`` that is a
  path to a local ``.txt`` / ``.json`` / ``.jsonl`` file is read with the matching ``datasets`` builder, and
  ``tokenizer_name == "bytes"`` selects :class:`ByteTokenizer`, so that real text can be trained on with no network.

Batches are produced in pinned host memory when a CUDA device is the target so that the ``.to(device,
non_blocking=True)`` copies in the train step overlap with compute.
"""
from __future__ import annotations

from functools import partial
from typing import Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import process_group_manager as pgm
from .utils import print


class SyntheticTokenDataset:
    """``num_samples`` windows of ``window`` uniform-random ids in ``[0, vocab_size)``; O(1) memory."""

    def __init__(self, num_samples: int, window: int, vocab_size: int, seed: int = 42):
        self.num_samples, self.window, self.vocab_size, self.seed = num_samples, window, vocab_size, seed

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        gen = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        return {"input_ids": torch.randint(0, self.vocab_size, (self.window,), generator=gen, dtype=torch.int64)}


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255 (``vocab_size >= 256``): the offline stand-in for a HF tokenizer."""

    vocab_size = 256

    def __call__(self, texts, return_attention_mask=False, return_token_type_ids=False):
        return {"input_ids": [list(t.encode("utf-8")) for t in texts]}

    def decode(self, ids) -> str:
        return bytes(int(i) for i in ids).decode("utf-8", errors="replace")


_LOCAL_BUILDERS = {".txt": "text", ".json": "json", ".jsonl": "json"}


class _ListDataset:
    def __init__(self, rows):
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, idx):
        return {"input_ids": torch.as_tensor(self.rows[idx], dtype=torch.int64)}


class MicroBatchDataLoader:
    def __init__(self, micro_batch_size, seq_length, dataset_name, tokenizer_name, num_workers, num_proc,
                 grad_acc_steps, device, subset_name=None, split="train", num_samples=None, pin_memory=True,
                 vocab_size: Optional[int] = None, seed: int = 42):
        g = pgm.get()
        self.micro_batch_size = micro_batch_size
        self.seq_length = seq_length
        self.grad_acc_steps = grad_acc_steps
        self.global_batch_size = micro_batch_size * grad_acc_steps * g.dp_world_size
        self.num_global_micro_batches = self.global_batch_size // self.micro_batch_size
        self.seq_length_per_gpu = seq_length // g.cp_world_size
        self.device = device
        self.pin_memory = bool(pin_memory) and torch.cuda.is_available() and \
            torch.device(device).type == "cuda"
        self.dp_rank, self.dp_world_size, self.cp_rank = g.dp_rank, g.dp_world_size, g.cp_rank

        if dataset_name == "synthetic":
            assert vocab_size is not None, "the synthetic dataset needs vocab_size"
            n = num_samples if num_samples else 1 << 30
            self.tokenized_dataset = SyntheticTokenDataset(n, seq_length + 1, vocab_size, seed)
            self.tokenizer = None
        else:
            self.tokenized_dataset = self._load_hf(dataset_name, tokenizer_name, subset_name, split, num_samples,
                                                   num_proc, device)
        self.epoch = 0
        self._cursor = 0
        # DistributedSampler(shuffle=False) semantics: pad to a multiple of dp, rank r takes r, r+dp, ...
        n = len(self.tokenized_dataset)
        self._samples_per_rank = (n + self.dp_world_size - 1) // self.dp_world_size
        # every micro-batch is full (the tail that does not fill one is dropped): pipeline messages, CUDA-graph inputs and
        # the symmetric workspaces are sized for exactly [micro_batch_size, seq_length_per_gpu]
        self._num_batches = self._samples_per_rank // micro_batch_size
        if n > 0 and self._num_batches == 0:
            raise ValueError(f"the dataset gives {self._samples_per_rank} samples per data-parallel rank, fewer than one "
                             f"micro-batch of {micro_batch_size}")

    # ------------------------------------------------------------------ HF path
    def _load_hf(self, dataset_name, tokenizer_name, subset_name, split, num_samples, num_proc, device):
        import os
        from datasets import load_dataset
        g = pgm.get()
        ext = os.path.splitext(str(dataset_name))[1].lower()
        if ext in _LOCAL_BUILDERS and os.path.exists(dataset_name):
            dataset = load_dataset(_LOCAL_BUILDERS[ext], data_files=str(dataset_name), split=split)
        else:
            dataset = load_dataset(dataset_name, split=split, name=subset_name)
        if g.global_rank == 0:
            print(f"rank {g.global_rank}: Creating tokenizer")
            if tokenizer_name == "bytes":
                objects = [ByteTokenizer()]
            else:
                from transformers import AutoTokenizer
                objects = [AutoTokenizer.from_pretrained(tokenizer_name)]
        else:
            objects = [None]
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast_object_list(objects, src=0, device=device)
        self.tokenizer = objects[0]
        if num_samples:
            dataset = dataset.select(range(min(num_samples, len(dataset))))
        return self.tokenize_dataset(dataset, "text", self.seq_length, num_proc)

    @staticmethod
    def tokenizer_group_text(examples, tokenizer, sequence_length):
        """Tokenise a list of texts, concatenate, cut into ``sequence_length + 1`` windows (stride ``sequence_length``)."""
        enc = tokenizer(examples, return_attention_mask=False, return_token_type_ids=False)
        ids = np.concatenate([np.asarray(x, dtype=np.int64) for x in enc["input_ids"]])
        return {"input_ids": group_into_windows(ids, sequence_length)}

    def tokenize_dataset(self, dataset, text_column_name, sequence_length, num_proc):
        from datasets import Features, Sequence, Value
        fn = partial(self.tokenizer_group_text, tokenizer=self.tokenizer, sequence_length=sequence_length)
        return dataset.map(
            fn, input_columns=text_column_name, remove_columns=dataset.column_names,
            features=Features({"input_ids": Sequence(feature=Value(dtype="int64"), length=sequence_length + 1)}),
            batched=True, num_proc=num_proc, load_from_cache_file=True,
            desc=f"Grouping texts in chunks of {sequence_length + 1}")

    # ------------------------------------------------------------------ batching
    def _sample_index(self, i: int) -> int:
        n = len(self.tokenized_dataset)
        return (self.dp_rank + i * self.dp_world_size) % n

    def collate_batch(self, batch) -> Dict[str, Optional[torch.Tensor]]:
        ids = torch.stack([torch.as_tensor(item["input_ids"]) for item in batch])
        bsz = ids.size(0)
        # the tokens of this context-parallel rank: one contiguous chunk (the reference's layout, data.py:105-108) or, with
        # distributed.cp_layout = "zigzag", an early and a late half-chunk (parallel/context_parallel.py)
        from .parallel.context_parallel import local_token_positions
        pos = local_token_positions(self.seq_length, self.cp_rank, self.seq_length // self.seq_length_per_gpu)
        input_ids = ids[:, pos].contiguous()
        target_ids = ids[:, pos + 1].contiguous()
        position_ids = pos.to(torch.long).unsqueeze(0).expand(bsz, -1).contiguous()
        if self.pin_memory:
            input_ids, target_ids, position_ids = input_ids.pin_memory(), target_ids.pin_memory(), position_ids.pin_memory()
        return {"input_ids": input_ids, "target_ids": target_ids, "position_ids": position_ids, "hidden_states": None}

    def __iter__(self):
        return self

    def __len__(self):
        return self._num_batches

    def __next__(self):
        if self._num_batches == 0:
            raise StopIteration
        if self._cursor >= self._num_batches:
            self.epoch += 1
            self._cursor = 0
        first = self._cursor * self.micro_batch_size
        idxs = [self._sample_index(first + j) for j in range(self.micro_batch_size)
                if first + j < self._samples_per_rank]
        self._cursor += 1
        return self.collate_batch([self.tokenized_dataset[i] for i in idxs])

    def state_dict(self):
        """Position in the data: the per-rank batch cursor, plus the same position counted in samples over all
        data-parallel ranks so that a run resumed with another ``dp_size`` or micro-batch size continues where the
        global stream stopped."""
        return {"epoch": self.epoch, "cursor": self._cursor, "micro_batch_size": self.micro_batch_size,
                "dp_world_size": self.dp_world_size,
                "samples_seen": self._cursor * self.micro_batch_size * self.dp_world_size}

    def load_state_dict(self, state):
        self.epoch, self._cursor = state["epoch"], state["cursor"]
        same_layout = (state.get("micro_batch_size", self.micro_batch_size) == self.micro_batch_size
                       and state.get("dp_world_size", self.dp_world_size) == self.dp_world_size)
        if not same_layout and "samples_seen" in state:
            # another data-parallel size or micro-batch size: continue at the first batch that starts at or after the
            # global position (a partially consumed round of the new layout is skipped rather than repeated)
            per_round = self.micro_batch_size * self.dp_world_size
            self._cursor = -(-int(state["samples_seen"]) // per_round)


def group_into_windows(ids: np.ndarray, sequence_length: int):
    """Windows of ``sequence_length + 1`` tokens at stride ``sequence_length`` (``data.py:57-76``)."""
    total = len(ids)
    if total >= sequence_length + 1:
        total = ((total - 1) // sequence_length) * sequence_length + 1
    return [ids[i:i + sequence_length + 1] for i in range(0, total - sequence_length, sequence_length)]
