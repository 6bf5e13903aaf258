"""Command-line front end (``surogate <command> config.yaml``).  Parity: surogate/cli/."""
