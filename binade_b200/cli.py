"""Command line: `python -m binade_b200.cli pack ...` and `... unpack ...`."""

import sys


def main():
    commands = ("pack", "unpack")
    if len(sys.argv) < 2 or sys.argv[1] not in commands:
        sys.exit("usage: binade_b200 {pack,unpack} ...  (pack --help for options)")
    cmd = sys.argv.pop(1)
    sys.argv[0] = f"binade_b200 {cmd}"
    if cmd == "pack":
        from .pack import main as run
    else:
        from .unpack import main as run
    run()


if __name__ == "__main__":
    main()
