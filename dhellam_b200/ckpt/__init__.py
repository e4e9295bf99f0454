from .megatron import fold_map, load_checkpoint, read_latest_iteration, save_checkpoint  # noqa: F401
