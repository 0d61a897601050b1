"""``python -m nmoe.data.cli <command> ...`` -> ``nmoe_b200.data.cli.main``: the data commands under the module path that
job files written for the reference use (nmoe/data/cli.py:1421-1646).  No ``__init__.py`` here either: a namespace
portion cannot shadow another installation of a package of the same name."""
from nmoe_b200.data.cli import build_parser, main  # noqa: F401

if __name__ == "__main__":
  raise SystemExit(main())
