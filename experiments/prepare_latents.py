"""Turn Parquet shards of pre-computed VAE latents into the flat memory-mapped files ``train_dit.py`` reads.

    python experiments/prepare_latents.py --source /data/imagenet-latents [--target DIR]

Input: ``train-*.parquet`` with columns ``latent_mean``, ``latent_mean_flip`` (4x32x32 fp32 each, possibly as
nested lists) and ``label``.  Output in ``DIR`` (default ``<source>/mmap``): ``latents.f32``
([n, 2, 4, 32, 32]: mean, flipped mean), ``labels.i64`` ([n]) and ``metadata.json``.  No VAE runs here; the
posterior means are stored unscaled and the trainer multiplies by 0.18215.  (Role of the reference's
experiments/prepare_latents.py:20-48.)
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path


def flat_values(column):
    import pyarrow as pa
    array = column.combine_chunks() if hasattr(column, "combine_chunks") else column
    if isinstance(array, pa.ExtensionArray):
        array = array.storage
    while pa.types.is_list(array.type) or pa.types.is_large_list(array.type) or pa.types.is_fixed_size_list(array.type):
        array = array.flatten()
    return array.to_numpy(zero_copy_only=False)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--source", required=True)
    parser.add_argument("--target")
    parser.add_argument("--rows-per-read", type=int, default=512)
    args = parser.parse_args()
    import numpy
    import pyarrow.parquet as pq
    source = Path(args.source)
    shards = sorted(source.glob("train-*.parquet"))
    if not shards:
        raise SystemExit(f"no train-*.parquet under {source}")
    total = sum(pq.ParquetFile(shard).metadata.num_rows for shard in shards)
    target = Path(args.target) if args.target else source / "mmap"
    target.mkdir(parents=True, exist_ok=True)
    latents = numpy.memmap(target / "latents.f32", dtype="float32", mode="w+", shape=(total, 2, 4, 32, 32))
    labels = numpy.memmap(target / "labels.i64", dtype="int64", mode="w+", shape=(total,))
    written = 0
    for shard in shards:
        reader = pq.ParquetFile(shard)
        for batch in reader.iter_batches(batch_size=args.rows_per_read, columns=["latent_mean", "latent_mean_flip", "label"]):
            stop = written + batch.num_rows
            latents[written:stop, 0] = flat_values(batch.column(0)).reshape(-1, 4, 32, 32)
            latents[written:stop, 1] = flat_values(batch.column(1)).reshape(-1, 4, 32, 32)
            labels[written:stop] = flat_values(batch.column(2))
            written = stop
        print(json.dumps({"shard": shard.name, "samples": written, "total": total}), flush=True)
    latents.flush()
    labels.flush()
    revision = None
    marker = source / "download_complete.json"
    if marker.exists():
        revision = json.loads(marker.read_text()).get("revision")
    (target / "metadata.json").write_text(json.dumps(
        {"samples": total, "shape": [total, 2, 4, 32, 32], "dtype": "float32", "scale_factor": 0.18215,
         "posterior": "mean", "source_revision": revision}, indent=2))


if __name__ == "__main__":
    main()
