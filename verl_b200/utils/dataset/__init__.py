from .rl_dataset import RLHFDataset, SyntheticPromptDataset, collate_fn, create_rl_dataset, create_rl_sampler  # noqa: F401
