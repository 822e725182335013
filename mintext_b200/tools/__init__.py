"""Data-preparation command-line tools (run as ``python -m mintext_b200.tools.<name>``)."""
