# tune-recipe: distributed=true
"""LoRA fine-tuning on a weighted mixture of datasets.

    tune run --nproc_per_node 8 dev/lora_finetune_distributed_multi_dataset --config dev/11B_lora_multi_dataset

Parity: recipes/dev/lora_finetune_distributed_multi_dataset.py of the reference.  Config: ``datasets`` is a list of entries
``{source, subset, split, transform: {_component_: …}, weight}`` — each becomes an SFT dataset (``transform`` receives the model
transform); ``dataloader`` holds ``shuffle``, ``collate_fn``, ``packed`` and the mixture's ``stop_criterion`` / ``seed``.  The
mixture is :class:`torchtune_b200.datasets.InterleavedDataset`; everything else is the LoRA SFT engine.
"""
import os
import sys
from functools import partial

from torchtune_b200 import config
from torchtune_b200.config import DictConfig, OmegaConf
from torchtune_b200.config._resolve import get_component_from_path
from torchtune_b200.data import padded_collate_packed
from torchtune_b200.datasets import InterleavedDataset, PackedDataset
from torchtune_b200.datasets._sft import _load
from torchtune_b200.engine.dataloading import StatefulDataLoader, StatefulDistributedSampler
from torchtune_b200.engine.sft import SFTTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class _Transformed:
    def __init__(self, rows, transform):
        self.rows, self.transform = rows, transform

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.transform(self.rows[i])


class LoRAFinetuneRecipeDistributedMultiDataset(SFTTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        cfg = DictConfig(OmegaConf.to_container(cfg, resolve=False))
        dl = cfg.get("dataloader") or DictConfig({})
        # the shared engine reads these top-level keys
        cfg["dataset"] = cfg.get("datasets")
        cfg["shuffle"] = dl.get("shuffle", True)
        if dl.get("collate_fn"):
            cfg["collate_fn"] = dl.get("collate_fn")
        super().__init__(cfg, distributed=all(os.environ.get(k) for k in ("RANK", "WORLD_SIZE")), lora=True)
        self._dl_cfg = dl

    def _setup_data(self, cfg_datasets, shuffle, batch_size, collate_fn, loader_state):
        parts, weights = [], []
        packed = bool(self._dl_cfg.get("packed", False))
        for entry in cfg_datasets:
            entry = dict(OmegaConf.to_container(entry, resolve=True)) if not isinstance(entry, dict) else dict(entry)
            weights.append(float(entry.pop("weight", 1.0)))
            transform = config.instantiate(DictConfig(entry.pop("transform")), model_transform=self._tokenizer)
            source = entry.pop("source")
            if "subset" in entry:
                entry["name"] = entry.pop("subset")
            ds = _Transformed(_load(source, **entry), transform)
            if packed:
                ds = PackedDataset(ds, max_seq_len=self._tokenizer.max_seq_len)
            parts.append(ds)
        mix = InterleavedDataset(parts, weights, seed=int(self._dl_cfg.get("seed", 0) or 0), stop_criterion=self._dl_cfg.get("stop_criterion", "cycle_until_all_exhausted"))
        dp_size = self.parallel.dp_size if self.parallel is not None else 1
        dp_rank = self.parallel.dp_rank if self.parallel is not None else 0
        sampler = StatefulDistributedSampler(mix, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle, seed=0)
        if packed:
            fn = padded_collate_packed
        else:
            pad_id = getattr(self._tokenizer, "pad_id", 0)
            fn = partial(get_component_from_path(collate_fn), padding_idx=pad_id, ignore_idx=getattr(self._loss_fn, "ignore_index", -100))
        loader = StatefulDataLoader(mix, batch_size=batch_size, sampler=sampler, collate_fn=fn, drop_last=True, pin_memory=self._device.type == "cuda")
        if loader_state is not None:
            loader.load_state_dict(loader_state)
        return loader


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="LoRAFinetuneRecipeDistributedMultiDataset", cfg=cfg)
    recipe = LoRAFinetuneRecipeDistributedMultiDataset(cfg=cfg)
    recipe.setup(cfg=recipe.cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
