"""Debug tooling behind ``surogate debug``: weight audit, registry dump, activation / gradient statistics, diff against transformers."""
