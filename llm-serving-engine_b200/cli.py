"""``python -m llmserve_b200 <command> ...``: the commands of this package under one name, as the
reference has them under ``llmserve`` (src/llmserve/cli.py). A command's module is imported only
when that command runs, so ``--help`` needs no GPU."""

from __future__ import annotations

import argparse
import importlib
import sys


def _commands(sub) -> None:
    """Each command: its name, the module whose ``main(argv)`` runs it, one line of help."""
    for name, module, about in (
        ("generate", "llmserve_b200.generate_cli", "generate tokens or text from the command line"),
        ("random-model", "llmserve_b200.random_model_cli", "write a random-weights model folder"),
    ):
        sub.add_parser(name, help=about, add_help=False).set_defaults(module=module)


def main(argv: list[str] | None = None) -> None:
    parser = argparse.ArgumentParser(prog="llmserve_b200", description=__doc__.split(":")[1].strip())
    _commands(parser.add_subparsers(dest="command", metavar="<command>"))
    args, rest = parser.parse_known_args(sys.argv[1:] if argv is None else argv)
    if args.command is None:
        parser.print_help()
        sys.exit(1)
    importlib.import_module(args.module).main(rest)


if __name__ == "__main__":
    main()
