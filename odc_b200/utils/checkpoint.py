"""Save / load full model and optimizer state of an FSDP2 model whose shards live in the symmetric heap.

Also takes the fused-kernel decoder (:class:`odc_b200.parallel.FusedDecoderLM` + ``FusedOptimizer``), whose model
file has the same names and shapes as ``DecoderLM``'s, so a model checkpoint moves between the two engines.

Same capability as the reference's example ``Checkpointer`` (examples/FSDP2/checkpoint.py:38-210):
two interchangeable back ends — the distributed-checkpoint state-dict API, or explicit DTensor
``full_tensor`` / ``distribute_tensor`` — writing ``model_state_dict.pt`` / ``optim_state_dict.pt``
into a folder named by a millisecond timestamp.  The sharded DTensor layout is untouched by the
on-demand engine (a parameter's local tensor is a view of heap memory), so files are
interchangeable with stock FSDP2.  Load BEFORE ``patch_lazy_init`` takes effect (first forward);
after a later ``load_state_dict(assign=True)`` call :func:`odc_b200.fsdp.fsdp2.repin_sharded_params`.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist
from torch.distributed.checkpoint.state_dict import (StateDictOptions, get_model_state_dict, get_optimizer_state_dict,
                                                     set_model_state_dict, set_optimizer_state_dict)
from torch.distributed.tensor import DTensor, distribute_tensor

MODEL_FILE = "model_state_dict.pt"
OPTIM_FILE = "optim_state_dict.pt"
META_FILE = "meta.json"


class Checkpointer:
    def __init__(self, folder: str, dcp_api: bool = True):
        self.folder, self.dcp_api = folder, dcp_api
        self.last_training_time = self._latest()

    def _latest(self) -> Optional[str]:
        if not os.path.isdir(self.folder):
            return None
        runs = [d for d in os.listdir(self.folder) if d.isdigit() and
                os.path.exists(os.path.join(self.folder, d, MODEL_FILE))]
        return max(runs, key=int) if runs else None

    def is_empty(self) -> bool:
        return self.last_training_time is None

    # ------------------------------------------------------------------ load
    def load_meta(self) -> dict:
        """What ``save(..., meta=...)`` stored next to the newest checkpoint (e.g. the next step to run), or ``{}``."""
        if self.last_training_time is None:
            return {}
        path = os.path.join(self.folder, self.last_training_time, META_FILE)
        if not os.path.exists(path):
            return {}
        with open(path) as f:
            return json.load(f)

    def load_model(self, model) -> None:
        path = os.path.join(self.folder, self.last_training_time, MODEL_FILE)
        full = torch.load(path, mmap=True, weights_only=True, map_location="cpu")
        if hasattr(model, "load_full_state_dict"):  # fused-kernel decoder: whole tensors under DecoderLM's names
            model.load_full_state_dict(full)
            return
        if self.dcp_api:
            set_model_state_dict(model, full, options=StateDictOptions(full_state_dict=True, broadcast_from_rank0=True))
            return
        sharded = {}
        meta = model.state_dict()
        for name, t in full.items():
            ref = meta[name]
            sharded[name] = torch.nn.Parameter(distribute_tensor(t.to(ref.device), ref.device_mesh, ref.placements)) \
                if isinstance(ref, DTensor) else t
        model.load_state_dict(sharded, assign=True)

    def load_optim(self, model, opt) -> None:
        path = os.path.join(self.folder, self.last_training_time, OPTIM_FILE)
        full = torch.load(path, mmap=True, weights_only=True, map_location="cpu")
        if hasattr(opt, "load_full_state_dict"):  # FusedAdamW: same file format as torch.optim.AdamW
            opt.load_full_state_dict(full)
            return
        set_optimizer_state_dict(model, opt, full, options=StateDictOptions(full_state_dict=True,
                                                                           broadcast_from_rank0=True))

    # ------------------------------------------------------------------ save
    def _model_state(self, model):
        if hasattr(model, "full_state_dict"):  # fused-kernel decoder (collective); same names and shapes as DecoderLM
            return {k: v.cpu() for k, v in model.full_state_dict().items()}
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP1
        if isinstance(model, FSDP1):  # flat parameters: unshard, read the original parameters under their own names
            with FSDP1.summon_full_params(model, writeback=False):
                return {k: v.detach().cpu().clone() for k, v in model.named_parameters()}
        if self.dcp_api:
            return get_model_state_dict(model, options=StateDictOptions(full_state_dict=True, cpu_offload=True))
        out = {}
        for name, t in model.state_dict().items():
            full = t.full_tensor() if isinstance(t, DTensor) else t
            if not dist.is_initialized() or dist.get_rank() == 0:
                out[name] = full.cpu()
        return out

    def export_hf(self, model, cfg, path: str, dtype: torch.dtype = torch.bfloat16) -> None:
        """Write the model as a Hugging Face Llama / Qwen2 checkpoint folder (collective; rank 0 writes).

        ``cfg`` is the model's ``DecoderConfig``.  The result loads with ``AutoModelForCausalLM.from_pretrained``
        and with :func:`odc_b200.models.hf.load_hf_checkpoint`.
        """
        from ..models.hf import save_hf_checkpoint
        sd = self._model_state(model)
        if not dist.is_initialized() or dist.get_rank() == 0:
            save_hf_checkpoint(path, sd, cfg, dtype=dtype)
        if dist.is_initialized():
            dist.barrier()

    def save(self, model, optim=None, meta: Optional[dict] = None) -> str:
        model_sd = self._model_state(model)
        optim_sd = None
        if optim is not None and hasattr(optim, "full_state_dict"):
            optim_sd = optim.full_state_dict()  # FusedAdamW writes the layout torch.optim.AdamW has
        elif optim is not None:
            optim_sd = get_optimizer_state_dict(model, optim, options=StateDictOptions(full_state_dict=True,
                                                                                       cpu_offload=True))
        stamp = str(int(time.time() * 1000))
        if dist.is_initialized():
            box = [stamp]
            dist.broadcast_object_list(box, src=0)
            stamp = box[0]
        folder = os.path.join(self.folder, stamp)
        if not dist.is_initialized() or dist.get_rank() == 0:
            os.makedirs(folder, exist_ok=True)
            torch.save(model_sd, os.path.join(folder, MODEL_FILE))
            if optim_sd is not None:
                torch.save(optim_sd, os.path.join(folder, OPTIM_FILE))
            if meta is not None:
                with open(os.path.join(folder, META_FILE), "w") as f:
                    json.dump(meta, f)
        if dist.is_initialized():
            dist.barrier()
        self.last_training_time = stamp
        return folder
