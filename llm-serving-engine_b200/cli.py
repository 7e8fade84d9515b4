"""Command-line entry point: ``python -m llmserve_b200 <command> ...`` (src/llmserve/cli.py)."""

from __future__ import annotations

import importlib
import sys

COMMANDS = {
    "generate": ("llmserve_b200.generate_cli", "generate tokens or text from the command line"),
    "random-model": ("llmserve_b200.random_model_cli", "write a random-weights model folder"),
}


def main(argv: list[str] | None = None) -> None:
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] in ("-h", "--help") or argv[0] not in COMMANDS:
        print("usage: llmserve_b200 <command> [args]\n\ncommands:")
        for name, (_, helptext) in COMMANDS.items():
            print(f"  {name:14s} {helptext}")
        sys.exit(0 if argv and argv[0] in ("-h", "--help") else 1)
    importlib.import_module(COMMANDS[argv[0]][0]).main(argv[1:])


if __name__ == "__main__":
    main()
