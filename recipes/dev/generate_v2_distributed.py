# tune-recipe: distributed=true
"""Tensor-parallel generation: the model's weights are split over all ranks, every rank decodes the same sequence.

    tune run --nproc_per_node 8 dev/generate_v2_distributed --config llama3_1/70B_generation_distributed

Parity: recipes/dev/generate_v2_distributed.py:40-270 of the reference.  Each rank loads the checkpoint, keeps its slice of every
projection (heads / MLP columns), and runs attention on its own heads with its own KV cache; the two row-parallel projections of a
layer are summed over the ranks.  Sampling uses the same seed on every rank, so all ranks draw the same token.
"""
import sys
import time
from typing import List

import torch
import torch.distributed as dist

from torchtune_b200 import config, training, utils
from torchtune_b200.config import DictConfig, OmegaConf
from torchtune_b200.generation import sample
from torchtune_b200.parallel.tp import TensorParallelContext
from torchtune_b200.parallel.tp_model import tensor_parallelize

sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent))
from generate_v2 import SingleTurnYAMLToMessages  # noqa: E402


class InferenceRecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self._device)
        self._logger = utils.get_logger(cfg.get("log_level", "INFO"))
        if not dist.is_initialized():
            dist.init_process_group("nccl" if self._device.type == "cuda" else "gloo", **({"device_id": self._device} if self._device.type == "cuda" else {}))
        self._world, self._rank = utils.get_world_size_and_rank()
        seed = cfg.get("seed") if cfg.get("seed") is not None else 1234
        torch.manual_seed(int(seed))  # identical on all ranks: every rank must sample the same token

    def setup(self, cfg: DictConfig) -> None:
        ckpt = config.instantiate(cfg.checkpointer).load_checkpoint()
        with training.set_default_dtype(self._dtype), self._device:
            model = config.instantiate(cfg.model)
        model.load_state_dict(ckpt[training.MODEL_KEY])
        self._tp = TensorParallelContext(self._device, max_rows_per_rank=128, max_width=model.tok_embeddings.embedding_dim)
        self.model = tensor_parallelize(model.eval(), self._tp).eval()
        self.model_transform = config.instantiate(cfg.tokenizer)
        self.to_messages = SingleTurnYAMLToMessages()
        utils.log_rank_zero(self._logger, f"Model was initialized with precision {self._dtype} over {self._world} ranks.")

    @torch.inference_mode()
    def generate(self, cfg: DictConfig) -> str:
        messages = self.to_messages(OmegaConf.to_container(cfg.prompt))
        inputs = self.model_transform({"messages": messages}, inference=True)
        prompt = torch.tensor(inputs["tokens"], device=self._device).unsqueeze(0)
        seq_len = prompt.shape[1]
        total = seq_len + cfg.max_new_tokens
        with self._device:
            self.model.setup_caches(batch_size=1, dtype=self._dtype, decoder_max_seq_len=total)
        causal = torch.tril(torch.ones(total, total, dtype=torch.bool, device=self._device))
        positions = torch.arange(total, device=self._device)
        generated: List[int] = []
        t0 = time.perf_counter()
        logits = self.model.forward_inference(prompt, mask=causal[None, :seq_len], input_pos=positions[None, :seq_len])[:, -1]
        token = sample(logits, temperature=cfg.temperature, top_k=cfg.get("top_k"))
        generated.append(token.item())
        for _ in range(cfg.max_new_tokens - 1):
            if token.item() in self.model_transform.stop_tokens:
                break
            logits = self.model.forward_inference(token.view(1, 1), mask=causal[None, seq_len : seq_len + 1], input_pos=positions[None, seq_len : seq_len + 1])[:, -1]
            token = sample(logits, temperature=cfg.temperature, top_k=cfg.get("top_k"))
            generated.append(token.item())
            seq_len += 1
        if self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        dt = time.perf_counter() - t0
        text = self.model_transform.decode(generated)
        if self._rank == 0:
            self._logger.info(f"\n\n{text}\n")
            self._logger.info(f"Time for inference: {dt:.02f} sec total, {len(generated) / dt:.02f} tokens/sec")
        return text

    def cleanup(self) -> None:
        self._tp.close()
        dist.destroy_process_group()


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="InferenceRecipe", cfg=cfg)
    recipe = InferenceRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.generate(cfg=cfg)
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(main())
