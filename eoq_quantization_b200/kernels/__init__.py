"""Modules that mirror the reference's ``kernels/`` package where it is part of the hot path."""
