"""Command-line entry points (``python -m neuralfn_b200.cli.nfn``)."""
