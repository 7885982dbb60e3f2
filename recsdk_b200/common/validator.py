"""Chainable argument validators and ``*_safe_check`` helpers.
Reference: ``training/common/python/validator/validator.py`` (chain style), ``safe_checker.py:31-101``."""
from __future__ import annotations

import os
import re
from typing import Any, Callable, Iterable, List, Optional, Tuple


class ValidationError(ValueError):
    pass


class Validator:
    """``Validator(value, "name").check_type(int).check_range(1, 8).validate()``; checks run in order and the first
    failure raises ``ValidationError`` naming the argument."""

    def __init__(self, value: Any, name: str = "value") -> None:
        self.value, self.name = value, name
        self._checks: List[Tuple[Callable[[Any], bool], str]] = []

    def add(self, fn: Callable[[Any], bool], message: str) -> "Validator":
        self._checks.append((fn, message))
        return self

    def check_type(self, *types) -> "Validator":
        return self.add(lambda v: isinstance(v, types) and not (isinstance(v, bool) and bool not in types),
                        "must be of type %s" % "/".join(t.__name__ for t in types))

    def check_range(self, lo=None, hi=None) -> "Validator":
        return self.add(lambda v: (lo is None or v >= lo) and (hi is None or v <= hi), "must be in [%s, %s]" % (lo, hi))

    def check_in(self, options: Iterable) -> "Validator":
        opts = list(options)
        return self.add(lambda v: v in opts, "must be one of %s" % (opts,))

    def check_regex(self, pattern: str) -> "Validator":
        rx = re.compile(pattern)
        return self.add(lambda v: isinstance(v, str) and rx.match(v) is not None, "must match %r" % pattern)

    def check_length(self, lo: int = 0, hi: Optional[int] = None) -> "Validator":
        return self.add(lambda v: len(v) >= lo and (hi is None or len(v) <= hi), "length must be in [%s, %s]" % (lo, hi))

    def validate(self) -> Any:
        for fn, msg in self._checks:
            ok = False
            try:
                ok = bool(fn(self.value))
            except Exception:  # noqa: BLE001 - a failing predicate is a failed check
                ok = False
            if not ok:
                raise ValidationError("%s %s, got %r" % (self.name, msg, self.value))
        return self.value

    def is_valid(self) -> bool:
        try:
            self.validate()
            return True
        except ValidationError:
            return False


class StringValidator(Validator):
    def __init__(self, value: Any, name: str = "value", max_len: int = 1024) -> None:
        super().__init__(value, name)
        self.check_type(str).check_length(1, max_len)


class DirectoryValidator(StringValidator):
    """Path checks: no ``..`` traversal, optional existence / writability, and no symlinked final component."""

    def __init__(self, value: Any, name: str = "path", max_len: int = 4096) -> None:
        super().__init__(value, name, max_len)
        self.add(lambda v: ".." not in v.replace("\\", "/").split("/"), "must not contain '..'")

    def check_exists(self) -> "DirectoryValidator":
        self.add(os.path.isdir, "must be an existing directory")
        return self

    def check_not_symlink(self) -> "DirectoryValidator":
        self.add(lambda v: not os.path.islink(v.rstrip("/")), "must not be a symbolic link")
        return self

    def check_writable(self) -> "DirectoryValidator":
        self.add(lambda v: os.access(v if os.path.isdir(v) else os.path.dirname(os.path.abspath(v)) or ".", os.W_OK), "must be writable")
        return self


def int_safe_check(name: str, value: Any, lo: Optional[int] = None, hi: Optional[int] = None) -> int:
    return Validator(value, name).check_type(int).check_range(lo, hi).validate()


def float_safe_check(name: str, value: Any, lo: Optional[float] = None, hi: Optional[float] = None) -> float:
    return Validator(value, name).check_type(int, float).check_range(lo, hi).validate()


def str_safe_check(name: str, value: Any, pattern: Optional[str] = None, max_len: int = 1024) -> str:
    v = StringValidator(value, name, max_len)
    if pattern:
        v.check_regex(pattern)
    return v.validate()


def path_safe_check(name: str, value: Any, must_exist: bool = False) -> str:
    v = DirectoryValidator(value, name).check_not_symlink()
    if must_exist:
        v.check_exists()
    return v.validate()
