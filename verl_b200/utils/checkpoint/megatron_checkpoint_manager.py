"""Checkpoint manager of the tensor x pipeline x expert parallel engine, layout schema v2:

    <role>/
      ckpt_contents.json          manifest: every saved content -> path + format; written last, so it also marks completeness
      transformer_config.json     architecture and parallel layout (with ``extra``)
      model/huggingface/          config.json (+ merged HF weights with ``hf_model``)
      model/dist_ckpt/mp_rank_TT_PPP[_EEE]/model.pt        local shards under their full-model names (with ``model``)
      optimizer/dist_ckpt/mp_rank_TT_PPP[_EEE]/optim_dpD.pt   fp32 masters + Adam moments of this rank's optimizer shard
      extra/dist_ckpt/mp_rank_TT_PPP[_EEE]/extra_dpD.pt    random-number generator states, schedule position

``verl_b200.model_merger`` (backend ``megatron``) folds ``model/dist_ckpt`` back into one HuggingFace model. A directory
in the flat layout that preceded this schema (``mp_rank_*`` directly under the role directory) is refused at load time;
``migrate_layout`` (also ``python -m verl_b200.utils.checkpoint.megatron_checkpoint_manager <dir>``) converts it in place
with hard links.

Parity target: ``verl/utils/checkpoint/megatron_checkpoint_manager.py``, ``docs/advance/checkpoint.rst`` ("layout schema v2").
"""

from __future__ import annotations

import json
import os
import re
from typing import Optional

import torch
import torch.distributed as dist

from .checkpoint_manager import BaseCheckpointManager

__all__ = ["MegatronCheckpointManager", "migrate_layout", "SCHEMA_VERSION", "MANIFEST"]

SCHEMA_VERSION = 2
MANIFEST = "ckpt_contents.json"
_RANK_DIR = re.compile(r"mp_rank_(\d+)_(\d+)(?:_(\d+))?$")


def rank_dir(tp_rank: int, pp_rank: int, ep_rank: int = 0, ep: int = 1) -> str:
    return f"mp_rank_{tp_rank:02d}_{pp_rank:03d}" + (f"_{ep_rank:03d}" if ep > 1 else "")


class MegatronCheckpointManager(BaseCheckpointManager):
    def __init__(self, engine, processing_class=None, checkpoint_config=None, role: str = "actor"):
        super().__init__(model=engine, processing_class=processing_class, checkpoint_config=checkpoint_config)
        self.engine, self.role = engine, role
        t = engine.topo
        self.tp_rank, self.pp_rank, self.dp_rank, self.ep_rank, self.ep = t.tp_rank, t.pp_rank, t.dp_rank, t.ep_rank, t.ep
        self._sub = rank_dir(self.tp_rank, self.pp_rank, self.ep_rank, self.ep)

    def _barrier(self) -> None:
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    # ------------------------------------------------------------------ save
    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None) -> None:
        eng = self.engine
        os.makedirs(local_path, exist_ok=True)
        contents: dict[str, dict] = {}
        # one writer per distinct model shard: data-parallel rank 0, or every expert-parallel rank for its own experts
        writes_model = self.dp_rank == 0 or self.ep > 1
        if self.should_save_model:
            d = os.path.join(local_path, "model", "dist_ckpt", self._sub)
            if writes_model:
                os.makedirs(d, exist_ok=True)
                shard = {k: v.detach().cpu() for k, v in eng.local_named_tensors()}
                shard["__shard_meta__"] = eng.shard_meta()  # where each tensor sits in the unsharded one (for the merger)
                torch.save(shard, os.path.join(d, "model.pt"))
            contents["model"] = {"path": "model/dist_ckpt", "format": "verl_b200_model_parallel_shards"}
        hf_dir = os.path.join(local_path, "model", "huggingface")
        full = eng.gather_full_params() if self.should_save_hf_model else None  # collective: every rank takes part
        if eng.global_rank == 0:
            eng.full_arch.save_pretrained(hf_dir)
            contents["hf_config"] = {"path": "model/huggingface", "format": "huggingface"}
            if full is not None:
                from ..model import save_hf_weights

                save_hf_weights(full, hf_dir)
                contents["hf_model"] = {"path": "model/huggingface", "format": "huggingface"}
            if self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
                self.processing_class.save_pretrained(hf_dir)
                contents["tokenizer"] = {"path": "model/huggingface", "format": "huggingface"}
        del full
        if self.should_save_optimizer and not eng.forward_only:
            d = os.path.join(local_path, "optimizer", "dist_ckpt", self._sub)
            os.makedirs(d, exist_ok=True)
            torch.save(eng.optimizer_state(), os.path.join(d, f"optim_dp{self.dp_rank}.pt"))
            contents["optimizer"] = {"path": "optimizer/dist_ckpt", "format": "verl_b200_model_parallel_shards"}
            contents["lr_scheduler"] = {"path": "optimizer/dist_ckpt", "format": "verl_b200_model_parallel_shards", "key": "sched_step"}
        if self.should_save_extra:
            d = os.path.join(local_path, "extra", "dist_ckpt", self._sub)
            os.makedirs(d, exist_ok=True)
            torch.save({"rng": self.get_rng_state(), "global_step": global_step}, os.path.join(d, f"extra_dp{self.dp_rank}.pt"))
            contents["rng_state"] = {"path": "extra/dist_ckpt", "format": "verl_b200_model_parallel_shards", "key": "rng"}
            if eng.global_rank == 0:
                t = eng.topo
                with open(os.path.join(local_path, "transformer_config.json"), "w") as f:
                    json.dump({"arch": eng.full_arch.to_hf_dict(), "tensor_model_parallel_size": t.tp, "pipeline_model_parallel_size": t.pp,
                               "expert_model_parallel_size": t.ep, "data_parallel_size": t.dp,
                               "virtual_pipeline_model_parallel_size": getattr(eng, "vpp_size", 1)}, f, indent=2)
                contents["transformer_config"] = {"path": "transformer_config.json", "format": "json"}
        self._barrier()  # every shard is on disk before the manifest says so
        if eng.global_rank == 0:
            t = eng.topo
            manifest = {
                "schema_version": SCHEMA_VERSION, "framework": "verl_b200.model_parallel", "role": self.role,
                "arch": (eng.full_arch.to_hf_dict().get("architectures") or [eng.full_arch.model_type])[0],
                "global_step": int(global_step), "world_size": t.tp * t.pp * t.dp,
                "backend": {"tensor_parallel": t.tp, "pipeline_parallel": t.pp, "expert_parallel": t.ep, "data_parallel": t.dp,
                            "value_head": bool(eng.value_head)},
                "save_contents": sorted(self._flags("save_contents")),
                "contents": contents,
                "directories": {
                    "model/huggingface": "HuggingFace-format artefacts: config.json, tokenizer files, merged weights when hf_model was saved",
                    "model/dist_ckpt": "one directory per model-parallel rank with its local shards (model.pt)",
                    "optimizer/dist_ckpt": "fp32 master weights, Adam moments and schedule position of every optimizer shard",
                    "extra/dist_ckpt": "random-number generator states"},
            }
            tmp = os.path.join(local_path, MANIFEST + ".tmp")
            with open(tmp, "w") as f:
                json.dump(manifest, f, indent=2)
            os.replace(tmp, os.path.join(local_path, MANIFEST))
        self._barrier()
        self.register_checkpoint(local_path, max_ckpt_to_keep)

    # ------------------------------------------------------------------ load
    def load_checkpoint(self, local_path: Optional[str], hdfs_path: Optional[str] = None, del_local_after_load: bool = False) -> None:
        if local_path is None:
            return
        mpath = os.path.join(local_path, MANIFEST)
        if not os.path.exists(mpath):
            if os.path.isdir(local_path) and any(_RANK_DIR.match(d) for d in os.listdir(local_path)):
                raise RuntimeError(f"{local_path} holds a checkpoint in the flat layout that preceded schema v{SCHEMA_VERSION} "
                                   f"(mp_rank_* directories at its root). Convert it in place with "
                                   f"`python -m verl_b200.utils.checkpoint.megatron_checkpoint_manager {local_path}`")
            raise FileNotFoundError(f"{mpath} is missing: not a complete model-parallel checkpoint (the manifest is written last)")
        with open(mpath) as f:
            man = json.load(f)
        if int(man.get("schema_version", 0)) != SCHEMA_VERSION:
            raise RuntimeError(f"{mpath}: schema_version {man.get('schema_version')} is not {SCHEMA_VERSION}")
        b, t = man["backend"], self.engine.topo
        if (b["tensor_parallel"], b["pipeline_parallel"], b["expert_parallel"]) != (t.tp, t.pp, t.ep):
            raise RuntimeError(f"checkpoint was written with tp x pp x ep = {b['tensor_parallel']} x {b['pipeline_parallel']} x "
                               f"{b['expert_parallel']}, this job runs {t.tp} x {t.pp} x {t.ep}: merge it to HF weights and load those")

        def need(kind: str, fname: str) -> str:
            if kind not in man["contents"]:
                raise FileNotFoundError(f"load_contents asks for '{kind}', which {mpath} does not list (saved: {man['save_contents']})")
            path = os.path.join(local_path, man["contents"][kind]["path"], self._sub, fname)
            if not os.path.exists(path):
                raise FileNotFoundError(f"{path} is missing although the manifest lists '{kind}'")
            return path

        eng = self.engine
        if self.should_load_model:
            eng.load_local_named_tensors(torch.load(need("model", "model.pt"), map_location="cpu", weights_only=False))
        if self.should_load_optimizer and not eng.forward_only:
            if b["data_parallel"] != t.dp:
                raise RuntimeError(f"optimizer shards were written by {b['data_parallel']} data-parallel ranks, this job has {t.dp}")
            eng.load_optimizer_state(torch.load(need("optimizer", f"optim_dp{self.dp_rank}.pt"), map_location="cpu", weights_only=False))
        elif self.should_load_model and not eng.forward_only:
            eng.reset_master_from_params()
        if self.should_load_extra and b["data_parallel"] == t.dp:
            self.load_rng_state(torch.load(need("rng_state", f"extra_dp{self.dp_rank}.pt"), map_location="cpu", weights_only=False)["rng"])


def migrate_layout(path: str, copy: bool = False) -> dict:
    """Convert a role directory of the flat layout (``mp_rank_*/{model,optim_dp*,extra_dp*}.pt`` and ``huggingface/`` at its
    root) to schema v2 in place: files are hard-linked (or copied) into ``model|optimizer|extra/dist_ckpt`` and a manifest
    is written. Returns the manifest."""
    import shutil

    if os.path.exists(os.path.join(path, MANIFEST)):
        with open(os.path.join(path, MANIFEST)) as f:
            return json.load(f)
    ranks = [d for d in os.listdir(path) if _RANK_DIR.match(d)]
    if not ranks:
        raise FileNotFoundError(f"no mp_rank_* directories under {path}")
    place = shutil.copy2 if copy else os.link
    saved, tp, pp, ep, dp = set(), 0, 0, 0, 0
    for d in ranks:
        m = _RANK_DIR.match(d)
        tp, pp, ep = max(tp, int(m.group(1)) + 1), max(pp, int(m.group(2)) + 1), max(ep, int(m.group(3) or 0) + 1)
        for f in os.listdir(os.path.join(path, d)):
            kind = "model" if f == "model.pt" else "optimizer" if f.startswith("optim_dp") else "extra" if f.startswith("extra_dp") else None
            if kind is None:
                continue
            if kind != "model":
                dp = max(dp, int(re.search(r"dp(\d+)", f).group(1)) + 1)
            dst = os.path.join(path, kind, "dist_ckpt", d)
            os.makedirs(dst, exist_ok=True)
            if not os.path.exists(os.path.join(dst, f)):
                place(os.path.join(path, d, f), os.path.join(dst, f))
            saved.add(kind)
    if os.path.isdir(os.path.join(path, "huggingface")):
        os.makedirs(os.path.join(path, "model"), exist_ok=True)
        if not os.path.exists(os.path.join(path, "model", "huggingface")):
            shutil.copytree(os.path.join(path, "huggingface"), os.path.join(path, "model", "huggingface"),
                            copy_function=shutil.copy2 if copy else os.link)
    fmt = "verl_b200_model_parallel_shards"
    contents = {k: {"path": f"{k}/dist_ckpt", "format": fmt} for k in sorted(saved) if k != "extra"}
    if "extra" in saved:
        contents["rng_state"] = {"path": "extra/dist_ckpt", "format": fmt, "key": "rng"}
    if os.path.isdir(os.path.join(path, "model", "huggingface")):
        contents["hf_config"] = {"path": "model/huggingface", "format": "huggingface"}
    manifest = {"schema_version": SCHEMA_VERSION, "framework": "verl_b200.model_parallel", "role": os.path.basename(os.path.normpath(path)),
                "global_step": None, "world_size": tp * pp * max(dp, 1),
                "backend": {"tensor_parallel": tp, "pipeline_parallel": pp, "expert_parallel": ep, "data_parallel": max(dp, 1)},
                "save_contents": sorted(saved), "contents": contents, "migrated_from": "flat layout"}
    with open(os.path.join(path, MANIFEST), "w") as f:
        json.dump(manifest, f, indent=2)
    return manifest


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="convert a model-parallel checkpoint directory of the flat layout to schema v2")
    ap.add_argument("checkpoint", help="role directory, e.g. .../global_step_100/actor")
    ap.add_argument("--copy", action="store_true", help="copy files instead of hard-linking them")
    a = ap.parse_args()
    print(json.dumps(migrate_layout(a.checkpoint, a.copy), indent=2))
