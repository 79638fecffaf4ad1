"""Dataset loading for ``areno train``.

``--dataset-path`` accepts a raw file (json / jsonl / parquet / csv / tsv / arrow), a directory
(``save_to_disk`` output or a folder of raw files) or a Hugging Face reference
``repo[:config[:split]]``.  ``--dataset-loader-fn file.py[:fn]`` names a user function
``fn(dataset_path, *, default_loader, load_dataset, load_from_disk)`` that returns the rows
(default name ``load_training_dataset``).  Behaviour of ``areno/cli/train.py:805-939`` in the
reference.
"""

from __future__ import annotations

import importlib.util
from pathlib import Path

SUPPORTED_SUFFIXES = {".json", ".jsonl", ".parquet", ".csv", ".tsv", ".arrow"}
_BUILDERS = {".json": "json", ".jsonl": "json", ".parquet": "parquet", ".csv": "csv", ".tsv": "csv", ".arrow": "arrow"}


def split_loader_fn_spec(spec_text: str) -> tuple[Path, str]:
    if ":" in spec_text:
        path_text, fn_name = spec_text.rsplit(":", 1)
        if not path_text or not fn_name:
            raise ValueError(f"Invalid --dataset-loader-fn value: {spec_text}")
        return Path(path_text).resolve(), fn_name
    return Path(spec_text).resolve(), "load_training_dataset"


def load_dataset_loader_fn(spec_text: str):
    path, fn_name = split_loader_fn_spec(spec_text)
    spec = importlib.util.spec_from_file_location(f"areno_dataset_loader_{abs(hash(str(path)))}", path)
    if spec is None or spec.loader is None:
        raise ImportError(f"Could not load dataset loader from {path}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    fn = getattr(module, fn_name, None)
    if fn is None:
        raise AttributeError(f"{path} must define {fn_name}(...)")
    if not callable(fn):
        raise TypeError(f"{path}:{fn_name} is not callable")
    return fn


def builder_for_suffix(suffix: str) -> str:
    try:
        return _BUILDERS[suffix.lower()]
    except KeyError:
        raise ValueError(f"Unsupported dataset file suffix for --dataset-path: {suffix}") from None


def _train_split(dataset):
    if hasattr(dataset, "keys") and "train" in dataset:
        return dataset["train"]
    return dataset


def _read_parquet_plain(data_files):
    """Parquet files whose embedded HF feature metadata cannot be decoded: go through pandas."""
    import pandas as pd
    from datasets import Dataset

    files = data_files if isinstance(data_files, list) else [data_files]
    frames = [pd.read_parquet(f) for f in files]
    df = pd.concat(frames, ignore_index=True) if len(frames) > 1 else frames[0]
    return Dataset.from_pandas(df, preserve_index=False)


def _load_raw(builder: str, data_files, load_dataset):
    try:
        return load_dataset(builder, data_files=data_files, split="train")
    except TypeError:
        if builder != "parquet":
            raise
        return _read_parquet_plain(data_files)


def load_hf_dataset_ref(ref: str, load_dataset):
    parts = ref.split(":")
    if len(parts) > 3 or not parts[0]:
        raise ValueError(f"Invalid Hugging Face dataset reference for --dataset-path: {ref}")
    name = parts[0]
    config = parts[1] if len(parts) >= 2 and parts[1] else None
    split = parts[2] if len(parts) == 3 and parts[2] else "train"
    if config is not None:
        return load_dataset(name, config, split=split)
    try:
        return load_dataset(name, split=split)
    except ValueError as exc:
        # datasets that need a config but expose the usual default as "main" (e.g. gsm8k)
        if "Config name is missing" not in str(exc) or "'main'" not in str(exc):
            raise
        return load_dataset(name, "main", split=split)


def load_dataset_from_path(dataset_path: str, *, load_dataset, load_from_disk):
    path = Path(dataset_path)
    if path.is_dir():
        try:
            return _train_split(load_from_disk(str(path)))
        except Exception:
            files = sorted(str(p) for p in path.iterdir() if p.is_file() and p.suffix.lower() in SUPPORTED_SUFFIXES)
            if not files:
                raise
            return _load_raw(builder_for_suffix(Path(files[0]).suffix), files, load_dataset)
    if path.exists() or path.suffix.lower() in SUPPORTED_SUFFIXES:
        return _load_raw(builder_for_suffix(path.suffix), str(path), load_dataset)
    return load_hf_dataset_ref(dataset_path, load_dataset)


def load_dataset_for_training(dataset_path: str, *, dataset_loader_fn: str | None, load_dataset=None,
                              load_from_disk=None):
    if load_dataset is None or load_from_disk is None:
        import datasets

        load_dataset = load_dataset or datasets.load_dataset
        load_from_disk = load_from_disk or datasets.load_from_disk

    def default_loader(p):
        return load_dataset_from_path(p, load_dataset=load_dataset, load_from_disk=load_from_disk)

    if dataset_loader_fn is not None:
        fn = load_dataset_loader_fn(dataset_loader_fn)
        return fn(dataset_path, default_loader=default_loader, load_dataset=load_dataset, load_from_disk=load_from_disk)
    return default_loader(dataset_path)
