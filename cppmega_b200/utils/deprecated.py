"""Fail-closed gate for deprecated code paths: they run only when the caller acknowledges them explicitly
(the reference's ``require_deprecated_ack``, cppmega/megatron/deprecated_paths.py:11-33, with the
acknowledgement passed as an argument instead of read from the environment)."""
from __future__ import annotations


class DeprecatedPathError(RuntimeError):
    pass


def require_deprecated_ack(feature: str, acknowledged: bool, replacement: str = "", reason: str = "") -> None:
    if acknowledged:
        return
    msg = f"{feature} is deprecated and disabled"
    if reason:
        msg += f" ({reason})"
    if replacement:
        msg += f"; use {replacement}"
    msg += ". Pass acknowledge_deprecated=True to run it anyway."
    raise DeprecatedPathError(msg)
