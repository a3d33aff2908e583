from maester_b200.sft.dataset import (  # noqa: F401
    ConversationParquetDataset,
    build_sft_data_loader,
    mask_labels,
    packed_collate_fn,
    tokenize_conversation,
)
from maester_b200.sft.packed_dataset import PackedSFTDataset, create_packed_dataloader  # noqa: F401
