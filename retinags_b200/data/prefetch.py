"""Input pipeline: decode the images of the coming batches while the current step runs.

The reference feeds its training loop from ``DataLoader(GroupedItems(...), num_workers=8, prefetch_factor=2,
pin_memory=True)`` (``trainer4tree_partition.py:600-601``): worker processes decode the PNG/JPEG targets and pickle whole
cameras back.  Here the cameras of a batch are built by a small pool of threads that stays ``depth`` batches ahead of
the consumer: image decoding (PIL) and the copy into pinned memory release the interpreter lock, nothing is pickled,
and decoded images land in the dataset's pinned cache, so that later epochs skip the decode altogether.  The iterator
yields batches strictly in the order of ``groups``; an exception of a worker is raised at the batch it belongs to.
"""
from __future__ import annotations

from collections import deque
from concurrent.futures import ThreadPoolExecutor


class BatchPrefetcher:
    def __init__(self, dataset, groups, depth: int = 2, workers: int = 8):
        self.dataset, self.groups = dataset, [tuple(g) for g in groups]
        self.depth, self.workers = max(0, int(depth)), max(1, int(workers))

    def __len__(self):
        return len(self.groups)

    def __iter__(self):
        if self.depth == 0:  # synchronous: decode in the consuming thread
            for ids in self.groups:
                yield ids, [self.dataset[i] for i in ids]
            return
        pool = ThreadPoolExecutor(max_workers=self.workers, thread_name_prefix="rgs-prefetch")
        try:
            pending: deque = deque()
            nxt = 0

            def top_up():
                nonlocal nxt
                while nxt < len(self.groups) and len(pending) <= self.depth:
                    ids = self.groups[nxt]
                    pending.append((ids, [pool.submit(self.dataset.__getitem__, i) for i in ids]))
                    nxt += 1

            top_up()
            while pending:
                ids, futs = pending.popleft()
                cams = [f.result() for f in futs]
                top_up()
                yield ids, cams
        finally:
            pool.shutdown(wait=False, cancel_futures=True)
