"""Glue for third-party training stacks."""
