"""Configuration: flag table, config-format registry and scaling rules."""
from . import flags
from .scaling import apply_scaling_rule, compute_dimensions, compute_lr

CONFIG_FORMAT_TO_MODULE_MAP = {"base": flags}


def parse_args_with_format(format, base_parser, args, namespace):
    return CONFIG_FORMAT_TO_MODULE_MAP[format].parse_args(base_parser, args, namespace)


def registered_formats():
    return CONFIG_FORMAT_TO_MODULE_MAP.keys()
