"""``python -m lbann_b200.help``: print every command-line flag and option of the driver with
its type, default and environment variable (the reference's ``lbann_help`` executable,
src/drivers/lbann_help.cpp)."""
from .utils import options as opts


def main() -> int:
    print("usage: python -m lbann_b200.driver --prototext=<file> [options]")
    print(opts.Options().describe())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
