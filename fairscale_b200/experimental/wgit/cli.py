"""``wgit`` command line: one sub-command per repository operation.

The sub-commands, their arguments and what they print are those of fairscale/experimental/wgit/cli.py:13-108 (``init``,
``status``, ``version``, ``add FILE [--no_per_tensor]``, ``commit -m MESSAGE``, ``checkout REVISION``, ``log [-f FILE]``);
here each command is a row of a table: its help text, its arguments, and the function that runs it in the repository of the
current directory.
"""

import argparse
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

from . import Repo
from .version import __version_tuple__


def _here(init: bool = False) -> Repo:
    return Repo(Path.cwd(), init=init)


def _cmd_init(args: argparse.Namespace) -> None:
    _here(init=True)


def _cmd_status(args: argparse.Namespace) -> None:
    print(_here().status())


def _cmd_version(args: argparse.Namespace) -> None:
    print(".".join(str(part) for part in __version_tuple__))


def _cmd_add(args: argparse.Namespace) -> None:
    _here().add(args.add, per_tensor=not args.no_per_tensor)


def _cmd_commit(args: argparse.Namespace) -> None:
    _here().commit(args.message)


def _cmd_checkout(args: argparse.Namespace) -> None:
    _here().checkout(args.checkout)


def _cmd_log(args: argparse.Namespace) -> None:
    _here().log(args.file)


Argument = Tuple[Tuple[str, ...], Dict[str, Any]]
# name -> (description, arguments, action)
COMMANDS: Dict[str, Tuple[str, List[Argument], Callable[[argparse.Namespace], None]]] = {
    "init": ("Initialize a weigit repo", [], _cmd_init),
    "status": ("Shows the repo's current status", [], _cmd_status),
    "version": ("Print the version", [], _cmd_version),
    "add": ("add a file to the staged changeset (default: none)", [
        (("add",), dict(type=str, metavar="FILE_PATH", help="add a file to the staged changeset (default: none)")),
        (("--no_per_tensor",), dict(action="store_true", help="store the file as one blob")),
    ], _cmd_add),
    "commit": ("Commits the staged changes", [
        (("commit",), dict(action="store_true", help="Commit the staged changes")),
        (("-m", "--message"), dict(default="", type=str, required=True, help="commit message")),
    ], _cmd_commit),
    "checkout": ("checkout from a commit", [
        (("checkout",), dict(type=str, metavar="FILE_SHA1", help="checkout from a commit")),
    ], _cmd_checkout),
    "log": ("Show the history log of the repo or optionally of a file.", [
        (("--file", "-f"), dict(type=str, default="", help="Show the log of the file")),
    ], _cmd_log),
}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="WeiGit: A git-like tool for model weight tracking")
    commands = parser.add_subparsers(dest="command")
    for name, (description, arguments, _) in COMMANDS.items():
        sub = commands.add_parser(name, description=description)
        for flags, options in arguments:
            sub.add_argument(*flags, **options)
    return parser


def main(argv: Optional[List[str]] = None) -> None:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.command is None:
        parser.print_help()
        return
    COMMANDS[args.command][2](args)


if __name__ == "__main__":
    main()
