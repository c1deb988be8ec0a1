"""Rank-sharding of ordinary map-style ``DataLoader`` objects (viola/distributed/data.py:6-22)."""

from __future__ import annotations

from torch.utils.data import DataLoader, DistributedSampler, RandomSampler, SequentialSampler


def prepare_dataloader(loader, *, rank, world_size):
    """Return a loader whose sampler yields this rank's share.

    An existing ``DistributedSampler`` is passed through (after checking it matches this rank), a
    single-process run keeps the loader as is, and custom batch samplers / iterable datasets are
    rejected: those must be sharded by the training script.
    """
    if isinstance(loader.sampler, DistributedSampler):
        if loader.sampler.rank != rank or loader.sampler.num_replicas != world_size:
            raise ValueError("the loader's DistributedSampler belongs to a different rank / world size")
        return loader
    if world_size == 1:
        return loader
    if loader.batch_size is None or not isinstance(loader.sampler, (RandomSampler, SequentialSampler)):
        raise ValueError("custom batch samplers and iterable datasets must be sharded by the training script")
    sampler = DistributedSampler(loader.dataset, num_replicas=world_size, rank=rank,
                                 shuffle=isinstance(loader.sampler, RandomSampler), drop_last=loader.drop_last)
    options = dict(dataset=loader.dataset, batch_size=loader.batch_size, sampler=sampler,
                   num_workers=loader.num_workers, collate_fn=loader.collate_fn, pin_memory=loader.pin_memory,
                   drop_last=loader.drop_last, timeout=loader.timeout, worker_init_fn=loader.worker_init_fn,
                   generator=loader.generator, persistent_workers=loader.persistent_workers)
    if loader.num_workers:
        options.update(prefetch_factor=loader.prefetch_factor,
                       multiprocessing_context=loader.multiprocessing_context)
    return DataLoader(**options)
