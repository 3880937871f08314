"""Error values of the library.

The five codes are the ones the reference reports everywhere
(src/kidi/core/error.h:8-19); the command line maps them onto exit codes the
way src/kidi/cli/main.cpp:1028-1035 does (usage faults 2, everything else 1).
"""
from __future__ import annotations

import enum


class ErrorCode(enum.Enum):
    INVALID_ARGUMENT = "invalid_argument"
    IO = "io"
    INVALID_MANIFEST = "invalid_manifest"
    UNSUPPORTED = "unsupported"
    RUNTIME = "runtime"


class KidiError(Exception):
    """An error with one of the five codes and a message for a person."""

    def __init__(self, code: ErrorCode, message: str):
        super().__init__(f"{code.value}: {message}")
        self.code = code
        self.message = message


def invalid_argument(message: str) -> KidiError:
    return KidiError(ErrorCode.INVALID_ARGUMENT, message)


def io_error(message: str) -> KidiError:
    return KidiError(ErrorCode.IO, message)


def invalid_manifest(message: str) -> KidiError:
    return KidiError(ErrorCode.INVALID_MANIFEST, message)


def unsupported(message: str) -> KidiError:
    return KidiError(ErrorCode.UNSUPPORTED, message)


def runtime_error(message: str) -> KidiError:
    return KidiError(ErrorCode.RUNTIME, message)
