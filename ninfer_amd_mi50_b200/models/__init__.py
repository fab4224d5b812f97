from . import qwen2_moe, vekasun, difavik, fetezen, kopadra  # noqa: F401  (registration)
