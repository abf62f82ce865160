"""``wgit`` command line (parity: fairscale/experimental/wgit/cli.py:13-108)."""

import argparse
from pathlib import Path
from typing import List, Optional

from . import Repo
from .version import __version_tuple__


def main(argv: Optional[List[str]] = None) -> None:
    desc = "WeiGit: A git-like tool for model weight tracking"
    parser = argparse.ArgumentParser(description=desc)
    sub = parser.add_subparsers(dest="command")
    sub.add_parser("init", description="Initialize a weigit repo")
    sub.add_parser("status", description="Shows the repo's current status")
    sub.add_parser("version", description="Print the version")
    p = sub.add_parser("add", description="add a file to the staged changeset (default: none)")
    p.add_argument("add", type=str, metavar="FILE_PATH", help="add a file to the staged changeset (default: none)")
    p.add_argument("--no_per_tensor", action="store_true", help="store the file as one blob")
    p = sub.add_parser("commit", description="Commits the staged changes")
    p.add_argument("commit", action="store_true", help="Commit the staged changes")
    p.add_argument("-m", "--message", default="", type=str, required=True, help="commit message")
    p = sub.add_parser("checkout", description="checkout from a commit")
    p.add_argument("checkout", type=str, metavar="FILE_SHA1", help="checkout from a commit")
    p = sub.add_parser("log", description="Show the history log of the repo or optionally of a file.")
    p.add_argument("--file", "-f", type=str, default="", help="Show the log of the file")
    args = parser.parse_args(argv)
    if args.command == "init":
        Repo(Path.cwd(), init=True)
    elif args.command == "add":
        Repo(Path.cwd()).add(args.add, per_tensor=not args.no_per_tensor)
    elif args.command == "status":
        out = Repo(Path.cwd()).status()
        print(out)
    elif args.command == "log":
        Repo(Path.cwd()).log(args.file)
    elif args.command == "commit":
        Repo(Path.cwd()).commit(args.message)
    elif args.command == "checkout":
        Repo(Path.cwd()).checkout(args.checkout)
    elif args.command == "version":
        print(".".join(str(x) for x in __version_tuple__))
    else:
        parser.print_help()


if __name__ == "__main__":
    main()
