from . import qwen2_moe, vekasun, difavik, fetezen  # noqa: F401  (registration)
