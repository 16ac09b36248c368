from .base_model_merger import generate_config_from_args, parse_args


def main(argv=None):
    args = parse_args(argv)
    config = generate_config_from_args(args)
    print(f"config: {config}")
    if config.backend == "fsdp":
        from .fsdp_model_merger import FSDPModelMerger as Merger
    elif config.backend == "megatron":
        from .megatron_model_merger import MegatronModelMerger as Merger
    else:
        raise NotImplementedError(f"Unknown backend: {config.backend}")
    merger = Merger(config)
    merger.merge_and_save()
    merger.cleanup()


if __name__ == "__main__":
    main()
