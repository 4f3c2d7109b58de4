"""Environment every worker process of a PPO job starts with. Parity target: ``verl/trainer/constants_ppo.py``
(``PPO_RAY_RUNTIME_ENV``, ``get_ppo_ray_runtime_env``)."""

import os

PPO_RUNTIME_ENV = {
    "env_vars": {
        "TOKENIZERS_PARALLELISM": "true",
        "NCCL_DEBUG": "WARN",
        "CUDA_DEVICE_MAX_CONNECTIONS": "1",       # keeps compute/communication issue order deterministic for overlap
        "NCCL_CUMEM_ENABLE": "0",                 # avoid CUDA VMM pools competing with the KV-cache allocator
        "TORCH_NCCL_AVOID_RECORD_STREAMS": "1",
    }
}
PPO_RAY_RUNTIME_ENV = PPO_RUNTIME_ENV


def get_ppo_ray_runtime_env() -> dict:
    """The defaults above minus every variable the user already set (user settings win)."""
    env = {k: v for k, v in PPO_RUNTIME_ENV["env_vars"].items() if k not in os.environ}
    return {"env_vars": env}


def apply_runtime_env() -> None:
    for k, v in get_ppo_ray_runtime_env()["env_vars"].items():
        os.environ[k] = v
