from .dataset import (SyntheticTokenDataset, BaseTrainingDataset, StreamingBaseTrainingDataset, ConversationDataset,
                      InterleavedDataset, HybridDatasetManager, setup_datasets, create_dataloader, create_fast_dataloader, collate)
