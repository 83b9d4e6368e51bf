"""Dataset and data-loader construction (megatron/data/data_utils.py): single-path splits
(``split: "969,30,1"``), weighted blends of several paths (optionally weighted by document counts),
pairwise and online variants, the synthetic token source, resumption (``start_iter``) and infinite
iterators.  Only tensor-rank 0 of the first and last pipeline stage reads data; the do_train /
do_valid / do_test flags are broadcast to everyone."""
from __future__ import annotations

import math
from itertools import cycle, zip_longest
from typing import List, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..utils.common import print_rank_0
from .blendable_dataset import BlendableDataset
from .gpt2_dataset import GPT2Dataset
from .indexed_dataset import make_dataset as make_indexed_dataset
from .samplers import DistributedBatchSampler
from .synthetic import SyntheticDataset


def make_data_loader(dataset, neox_args):
    """Sequential sampling, one global batch cut into data-parallel slices."""
    if dataset is None:
        return None
    world_size = mpu.get_data_parallel_world_size()
    rank = mpu.get_data_parallel_rank()
    global_batch_size = neox_args.batch_size * world_size
    sampler = torch.utils.data.SequentialSampler(dataset)
    batch_sampler = DistributedBatchSampler(sampler=sampler, batch_size=global_batch_size, drop_last=True, rank=rank,
                                            world_size=world_size)
    return torch.utils.data.DataLoader(dataset, batch_sampler=batch_sampler, num_workers=neox_args.num_workers,
                                       pin_memory=True)


def _maybe(path, impl, skip_warmup):
    return make_indexed_dataset(path, impl, skip_warmup) if path is not None else None


def build_the_dataset(data_prefix, pos_data_prefix, neg_data_prefix, name, data_impl, pack_impl, dataset_impl,
                      allow_chopped, num_samples, num_epochs, seq_length, seed, skip_warmup, build_index_mappings=True,
                      label_prefix=None, pos_label_prefix=None, neg_label_prefix=None, precompute_model_name=None,
                      reward_prefix=None):
    """One dataset (gpt2 | pairwise) over one path, with its optional label / reward / reference streams."""
    if dataset_impl == "gpt2":
        indexed = make_indexed_dataset(data_prefix, data_impl, skip_warmup)
        label_ds = _maybe(label_prefix, data_impl, skip_warmup)
        reward_ds = _maybe(reward_prefix, data_impl, skip_warmup)
        ref_ds = _maybe(data_prefix + "_" + precompute_model_name, data_impl, skip_warmup) \
            if precompute_model_name is not None else None
        total = indexed.sizes.shape[0]
        print_rank_0("    {}:".format(name))
        print_rank_0("     no. of documents:{}".format(total))
        documents = np.arange(start=0, stop=total, step=1, dtype=np.int32)
        return GPT2Dataset(name, data_prefix, documents, indexed, num_samples, num_epochs, seq_length, seed,
                           pack_impl=pack_impl, allow_chopped=allow_chopped,
                           build_index_mappings=build_index_mappings, label_dataset=label_ds,
                           reward_dataset=reward_ds, ref_dataset=ref_ds)
    if dataset_impl == "pairwise":
        from .pairwise_dataset import PairwiseDataset
        pos = make_indexed_dataset(pos_data_prefix, data_impl, skip_warmup)
        neg = make_indexed_dataset(neg_data_prefix, data_impl, skip_warmup)
        pos_label = _maybe(pos_label_prefix, data_impl, skip_warmup)
        neg_label = _maybe(neg_label_prefix, data_impl, skip_warmup)
        pos_ref = neg_ref = None
        if precompute_model_name is not None:
            pos_ref = make_indexed_dataset(pos_data_prefix + "_" + precompute_model_name, data_impl, skip_warmup)
            neg_ref = make_indexed_dataset(neg_data_prefix + "_" + precompute_model_name, data_impl, skip_warmup)
        total = pos.sizes.shape[0]
        documents = np.arange(start=0, stop=total, step=1, dtype=np.int32)
        return PairwiseDataset(name, pos_data_prefix, documents, pos, neg, num_samples, seq_length, seed,
                               pack_impl=pack_impl, allow_chopped=allow_chopped,
                               build_index_mappings=build_index_mappings, pos_label_dataset=pos_label,
                               neg_label_dataset=neg_label, pos_ref_dataset=pos_ref, neg_ref_dataset=neg_ref)
    raise NotImplementedError(f"dataset_impl={dataset_impl} not implemented")


def get_train_valid_test_split_(splits_string, size):
    """"969,30,1" -> document index boundaries [0, a, b, size]."""
    if splits_string.find(",") != -1:
        splits = [float(s) for s in splits_string.split(",")]
    elif splits_string.find("/") != -1:
        splits = [float(s) for s in splits_string.split("/")]
    else:
        splits = [float(splits_string)]
    while len(splits) < 3:
        splits.append(0.0)
    splits = splits[:3]
    total = sum(splits)
    assert total > 0.0
    splits = [s / total for s in splits]
    idx = [0]
    for s in splits:
        idx.append(idx[-1] + int(round(s * float(size))))
    diff = idx[-1] - size
    for i in range(1, len(idx)):
        idx[i] -= diff
    assert len(idx) == 4 and idx[-1] == size
    return idx


def build_train_valid_test_datasets(data_prefix, use_shared_fs, data_impl, pack_impl, allow_chopped, splits_string,
                                    train_valid_test_num_samples, train_valid_test_epochs, seq_length, seed,
                                    skip_warmup):
    """Three GPT datasets over consecutive document ranges of one indexed file."""
    indexed = make_indexed_dataset(data_prefix, data_impl, skip_warmup)
    total = indexed.sizes.shape[0]
    splits = get_train_valid_test_split_(splits_string, total)
    print_rank_0(" > dataset split:")
    for i, n in enumerate(("train", "validation", "test")):
        print_rank_0("    {}:".format(n))
        print_rank_0("     document indices in [{}, {}) total of {} documents".format(
            splits[i], splits[i + 1], splits[i + 1] - splits[i]))

    def build(index, name):
        if splits[index + 1] <= splits[index]:
            return None
        documents = np.arange(start=splits[index], stop=splits[index + 1], step=1, dtype=np.int32)
        return GPT2Dataset(name, data_prefix, documents, indexed, train_valid_test_num_samples[index],
                           train_valid_test_epochs[index], seq_length, seed, pack_impl=pack_impl,
                           allow_chopped=allow_chopped, use_shared_fs=use_shared_fs)
    return build(0, "train"), build(1, "valid"), build(2, "test")


def get_normalized_weights_and_num_samples(weights: List[float], num_samples: int) -> Tuple[List[float], List[int]]:
    weight_sum = sum(weights)
    assert weight_sum > 0.0
    weights = [w / weight_sum for w in weights]
    if num_samples is not None:
        # a little over-provisioning so that rounding never starves a dataset
        return weights, [int(math.ceil(num_samples * w * 1.005)) for w in weights]
    return weights, [None] * len(weights)


def build_weighted_datasets(neox_args, train_num_samples, valid_num_samples, test_num_samples, train_epochs,
                            valid_epochs, test_epochs, build_index_mappings=True):
    """One dataset per configured path for each split."""
    def paths(kind, split):
        v = getattr(neox_args, f"{kind}{split}_data_paths" if kind in ("pos_", "neg_") else f"{split}_data_paths") \
            if kind != "label" else getattr(neox_args, f"{split}_label_data_paths")
        return v or []
    out = {"train": [], "valid": [], "test": []}
    nums = {"train": train_num_samples, "valid": valid_num_samples, "test": test_num_samples}
    epochs = {"train": train_epochs, "valid": valid_epochs, "test": test_epochs}
    for split in ("train", "valid", "test"):
        plain = getattr(neox_args, f"{split}_data_paths") or []
        labels = getattr(neox_args, f"{split}_label_data_paths") or []
        rewards = getattr(neox_args, f"{split}_reward_data_paths") or []
        pos = getattr(neox_args, f"pos_{split}_data_paths") or []
        neg = getattr(neox_args, f"neg_{split}_data_paths") or []
        pos_l = getattr(neox_args, f"pos_{split}_label_data_paths") or []
        neg_l = getattr(neox_args, f"neg_{split}_label_data_paths") or []
        for i, (p, l, r, pp, np_, pl, nl) in enumerate(zip_longest(plain, labels, rewards, pos, neg, pos_l, neg_l)):
            n = nums[split][i] if nums[split] is not None and i < len(nums[split]) else None
            if n is None and epochs[split] is None:
                continue
            out[split].append(build_the_dataset(
                data_prefix=p, name=f"{split}_{i}", data_impl=neox_args.data_impl, pack_impl=neox_args.pack_impl,
                allow_chopped=neox_args.allow_chopped, num_samples=n, num_epochs=epochs[split],
                seq_length=neox_args.seq_length, seed=neox_args.seed, skip_warmup=(not neox_args.mmap_warmup),
                build_index_mappings=build_index_mappings, label_prefix=l, dataset_impl=neox_args.dataset_impl,
                pos_data_prefix=pp, neg_data_prefix=np_, pos_label_prefix=pl, neg_label_prefix=nl,
                precompute_model_name=neox_args.precompute_model_name, reward_prefix=r))
    return out["train"], out["valid"], out["test"]


def weights_by_num_docs(l: list, alpha=0.3):
    """p(L) proportional to |L|^alpha, then multiplied by (1 - unbiased share) and renormalised:
    boosts small datasets (arXiv:1911.02116)."""
    if len(l) == 1:
        return [1.0]
    total_n_docs = sum(l)
    unbiased = [i / total_n_docs for i in l]
    probs = [i ** alpha for i in unbiased]
    total = sum(probs)
    probs = [i / total for i in probs]
    weights = [p * (1 - u) for p, u in zip(probs, unbiased)]
    total = sum(weights)
    return [i / total for i in weights]


def validate_train_epochs(neox_args):
    if neox_args.train_epochs is None:
        return
    if neox_args.train_epochs and neox_args.train_iters:
        raise ValueError("Cannot specify both train epochs and train iters simultaneously")
    if neox_args.pack_impl != "packed":
        raise ValueError("Packing implementations other than 'packed' are currently unsupported with train_epochs")
    if neox_args.weight_by_num_documents:
        raise ValueError("Weighting by number of documents is currently unsupported with train_epochs")
    if neox_args.train_data_weights and (not all(w == 1.0 for w in neox_args.train_data_weights)):
        raise ValueError("train_data_weights != None is currently unsupported with train_epochs")
    if neox_args.dataset_impl != "gpt2":
        raise ValueError("non gpt2 datasets are not currently unsupported with train_epochs")


def _blend(datasets, weights):
    return BlendableDataset(datasets, weights) if datasets else None


def build_train_valid_test_data_loaders(neox_args):
    """-> {"train": loader, "valid": loader, "test": loader}; sets ``do_train/do_valid/do_test``."""
    validate_train_epochs(neox_args)
    train_dataloader = valid_dataloader = test_dataloader = None
    print_rank_0("> building train, validation, and test datasets ...")
    if neox_args.is_pipe_parallel:
        is_first = mpu.get_pipe_parallel_rank() == 0
        is_last = mpu.get_pipe_parallel_rank() == mpu.get_pipe_parallel_world_size() - 1
        pipe_load = is_first or is_last
    else:
        pipe_load = True
    device = "cuda" if (dist.is_initialized() and dist.get_backend() == "nccl") else "cpu"
    if mpu.get_model_parallel_rank() == 0 and pipe_load:
        if neox_args.train_epochs:
            train_iters = None
            train_val_test_num_samples = [None, None, None]
            train_val_test_epochs = [neox_args.train_epochs, 1, 1]
        else:
            train_iters = neox_args.train_iters
            eval_iters = (train_iters // neox_args.eval_interval + 1) * neox_args.eval_iters
            test_iters = neox_args.eval_iters
            train_val_test_num_samples = [train_iters * neox_args.train_batch_size,
                                          eval_iters * neox_args.train_batch_size,
                                          test_iters * neox_args.train_batch_size]
            train_val_test_epochs = [None, None, None]
        if neox_args.dataset_impl == "synthetic":
            vocab = min(neox_args.synthetic_vocab_size, neox_args.padded_vocab_size)
            mk = lambda n, seed: SyntheticDataset(max(int(n or 1), 1), neox_args.seq_length, vocab, seed)
            n = train_val_test_num_samples
            train_ds, valid_ds, test_ds = mk(n[0], neox_args.seed), mk(n[1], neox_args.seed + 1), \
                mk(n[2], neox_args.seed + 2)
        elif neox_args.dataset_impl == "online":
            from .online_dataset import OnlineDataset
            n = train_val_test_num_samples
            mk = lambda num, name: OnlineDataset(num_samples=num, seq_length=neox_args.seq_length, name=name,
                                                 leave_one_out=neox_args.reinforce_leave_one_out,
                                                 dataserver_ips=neox_args.online_dataserver_ips,
                                                 dataserver_ports=neox_args.online_dataserver_ports)
            train_ds, valid_ds, test_ds = mk(n[0], "train"), mk(n[1], "valid"), mk(n[2], "test")
        elif neox_args.train_data_paths or neox_args.pos_train_data_paths:
            train_weights, train_num = get_normalized_weights_and_num_samples(
                neox_args.train_data_weights, train_val_test_num_samples[0])
            valid_weights, valid_num = get_normalized_weights_and_num_samples(
                neox_args.valid_data_weights, train_val_test_num_samples[1])
            test_weights, test_num = get_normalized_weights_and_num_samples(
                neox_args.test_data_weights, train_val_test_num_samples[2])
            tds, vds, teds = build_weighted_datasets(
                neox_args, train_num, valid_num, test_num, train_val_test_epochs[0], train_val_test_epochs[1],
                train_val_test_epochs[2], build_index_mappings=not neox_args.weight_by_num_documents)
            if neox_args.weight_by_num_documents:
                get_docs = lambda ds: [d.indexed_dataset.sizes.shape[0] for d in ds]
                fn = lambda x: weights_by_num_docs(x, alpha=neox_args.weighted_sampler_alpha)
                train_weights, valid_weights, test_weights = fn(get_docs(tds)), fn(get_docs(vds)), fn(get_docs(teds))
                train_weights, train_num = get_normalized_weights_and_num_samples(
                    train_weights, train_val_test_num_samples[0])
                valid_weights, valid_num = get_normalized_weights_and_num_samples(
                    valid_weights, train_val_test_num_samples[1])
                test_weights, test_num = get_normalized_weights_and_num_samples(
                    test_weights, train_val_test_num_samples[2])
                tds, vds, teds = build_weighted_datasets(
                    neox_args, train_num, valid_num, test_num, train_val_test_epochs[0], train_val_test_epochs[1],
                    train_val_test_epochs[2])
            train_ds, valid_ds, test_ds = _blend(tds, train_weights), _blend(vds, valid_weights), \
                _blend(teds, test_weights)
        else:
            train_ds, valid_ds, test_ds = build_train_valid_test_datasets(
                data_prefix=neox_args.data_path, use_shared_fs=neox_args.use_shared_fs,
                data_impl=neox_args.data_impl, pack_impl=neox_args.pack_impl, allow_chopped=neox_args.allow_chopped,
                splits_string=neox_args.split, train_valid_test_num_samples=train_val_test_num_samples,
                train_valid_test_epochs=train_val_test_epochs, seq_length=neox_args.seq_length,
                seed=neox_args.seed, skip_warmup=(not neox_args.mmap_warmup))
        train_dataloader = make_data_loader(train_ds, neox_args=neox_args)
        valid_dataloader = make_data_loader(valid_ds, neox_args=neox_args)
        test_dataloader = make_data_loader(test_ds, neox_args=neox_args)
        if neox_args.train_epochs:
            do_train = train_dataloader is not None
            do_valid = valid_dataloader is not None
            do_test = test_dataloader is not None
        else:
            do_train = train_dataloader is not None and neox_args.train_iters > 0
            do_valid = valid_dataloader is not None and neox_args.eval_iters > 0
            do_test = test_dataloader is not None and neox_args.eval_iters > 0
        flags = torch.tensor([int(do_train), int(do_valid), int(do_test)], dtype=torch.long, device=device)
    else:
        flags = torch.tensor([0, 0, 0], dtype=torch.long, device=device)
    if dist.is_initialized():
        if neox_args.is_pipe_parallel:
            dist.broadcast(flags, src=0)
        else:
            dist.broadcast(flags, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
    neox_args.do_train = bool(flags[0].item())
    neox_args.do_valid = bool(flags[1].item())
    neox_args.do_test = bool(flags[2].item())
    return {"train": train_dataloader, "valid": valid_dataloader, "test": test_dataloader}


def shift_and_wrap_data_loaders(neox_args, data_loaders, loop=True):
    """Fast-forward the samplers to the resume point and wrap the loaders into iterators."""
    train_dataloader, valid_dataloader, test_dataloader = data_loaders["train"], data_loaders["valid"], \
        data_loaders["test"]
    if train_dataloader is not None:
        train_dataloader.batch_sampler.start_iter = (neox_args.iteration * neox_args.gradient_accumulation_steps) % \
            len(train_dataloader)
        print_rank_0("setting training data start iteration to {}".format(train_dataloader.batch_sampler.start_iter))
    if valid_dataloader is not None:
        start_iter_val = ((neox_args.iteration * neox_args.gradient_accumulation_steps) // neox_args.eval_interval) * \
            neox_args.eval_iters
        valid_dataloader.batch_sampler.start_iter = start_iter_val % len(valid_dataloader)
        print_rank_0("setting validation data start iteration to {}".format(valid_dataloader.batch_sampler.start_iter))
    wrap = (lambda dl: cycle(dl)) if loop else (lambda dl: iter(dl))
    return tuple(wrap(dl) if dl is not None else None for dl in (train_dataloader, valid_dataloader, test_dataloader))


def compile_helper():
    from .helpers import compile_helper as c
    c()
