from maester_b200.models.moe.moe import FeedForward, GroupedExperts, MoE, MoEArgs, TokenChoiceTopKRouter, TokenReorderer  # noqa: F401
