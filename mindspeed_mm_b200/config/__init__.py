"""Three accepted configuration schemas, one internal representation each:

1. ``legacy.parse_legacy_args``  - Megatron flags + ``--mm-model/--mm-data/--mm-tool`` JSON (or YAML) files
2. ``legacy.yaml_to_argv``       - single YAML with ``gpt_args`` flattened to (1)
3. ``native.load_config``        - single YAML ``parallel/data/model/features/training/tools`` (+ ``a.b=c`` overrides)
"""
from .legacy import MMConfig, merge_mm_args, parse_legacy_args, yaml_to_argv  # noqa: F401
from .native import Arguments, load_config, match_modules, module_name_match  # noqa: F401
from .tree import ConfigNode, get_dtype  # noqa: F401
