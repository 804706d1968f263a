"""Argument helpers shared by the checkpoint tools.  The reference's tools take their arguments the way python-fire
does (``--input X --output Y --unflatten-weights True``, dashes or underscores); these helpers make an ``argparse``
parser take the same spellings next to this package's own."""
from __future__ import annotations

import argparse


def _both_spellings(*names):
    out = []
    for n in names:
        for variant in (n, "--" + n[2:].replace("-", "_")):
            if variant not in out:
                out.append(variant)
    return out


def _truth(text: str) -> bool:
    if text.lower() in ("true", "1", "yes"):
        return True
    if text.lower() in ("false", "0", "no"):
        return False
    raise argparse.ArgumentTypeError(f"expected True or False, got {text}")


def add_option(parser, *names, **kwargs):
    """An option under every given name, each with dashes and with underscores."""
    return parser.add_argument(*_both_spellings(*names), **kwargs)


def add_switch(parser, *names, default: bool = False, help: str = ""):
    """A boolean that is set by ``--flag``, ``--flag True`` or ``--flag=False``."""
    return parser.add_argument(*_both_spellings(*names), nargs="?", const=True, default=default, type=_truth, help=help)
