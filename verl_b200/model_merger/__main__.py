"""``python -m verl_b200.model_merger merge --backend fsdp --local_dir <ckpt>/actor --target_dir <out>``"""
from .base_model_merger import parse_args


def main(argv=None):
    cfg = parse_args(argv)
    if cfg.backend == "fsdp":
        from .fsdp_model_merger import FSDPModelMerger as M
    elif cfg.backend == "megatron":
        from .megatron_model_merger import MegatronModelMerger as M
    else:
        raise NotImplementedError(f"Unknown backend: {cfg.backend}")
    merger = M(cfg)
    merger.merge_and_save()
    merger.cleanup()


if __name__ == "__main__":
    main()
