"""B200 (sm_100a) fused GRPO / PPO-clip token loss: a drop-in for the loss region of
demon2036/MLLM-JAX's TrainGRPOModule (MLLM_JAX/train_modules/__init__.py:118-180).

Importing the package does not need a GPU or the built library; calling an operator does.
"""
from ._lib import GrpoError, LIB_PATH, launch_count  # noqa: F401
from .ops import (  # noqa: F401
    LossConfig,
    TokenLossProblem,
    grpo_token_loss,
    grpo_token_loss_flat,
    grpo_value_and_grad,
    sft_cross_entropy,
    token_logprobs,
)
from .linear_loss import linear_grpo_value_and_grad  # noqa: F401
from .train_module import (  # noqa: F401
    TrainGRPOModule,
    per_sample_entropy,
    ppo_actor_critic_terms,
    ppo_policy_terms,
    ppo_value_loss,
)

__all__ = [
    "GrpoError", "LIB_PATH", "LossConfig", "TokenLossProblem", "TrainGRPOModule", "grpo_token_loss",
    "grpo_token_loss_flat", "grpo_value_and_grad", "linear_grpo_value_and_grad", "launch_count", "per_sample_entropy", "ppo_actor_critic_terms", "ppo_policy_terms", "ppo_value_loss",
    "sft_cross_entropy",
    "token_logprobs",
]
