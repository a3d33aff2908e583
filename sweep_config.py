"""Example sweep: learning-rate scan of a small Llama with muP on synthetic data.

    python sweep.py submit sweep_config.py --dry-run
"""
from maester_b200.config import Config
from sweep import SweepConfig, SweepValues

sweep_name = "llama-mup-lr-sweep"

base_config = Config(
    wandb_project=sweep_name,  # summarize/plot read the W&B project named like the sweep
    model_name="llama3",
    flavor="sweep",
    num_nodes=1,
    train_batch_size=8,
    time="00-02:00:00",
    train_num_steps=2000,
    enable_checkpoint=False,
    enable_mup=True,
    model_width=512,
    ac_mode="none",
    data_parallel_shard_degree=8,
    synthetic_data=True,
    synthetic_vocab_size=32000,
)

config = SweepConfig(
    sweep_name=sweep_name,
    base_config=base_config,
    parameter_space={
        "opt_cfg.lr": SweepValues.logspace(-11, -7, 5, base=2),
    },
)
