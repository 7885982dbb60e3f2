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


def class_safe_check(name: str, value: Any, classes) -> Any:
    """``value`` must be an instance of ``classes`` (a class or a tuple of classes)."""
    classes = tuple(classes) if isinstance(classes, (list, tuple)) else (classes,)
    return Validator(value, name).add(lambda v: isinstance(v, classes), "must be an instance of %s"
                                      % "/".join(getattr(c, "__name__", str(c)) for c in classes)).validate()


def dir_safe_check(name: str, directory: Any) -> str:
    """An existing directory, given as a non-empty path of bounded length without ``..`` and not through a symbolic link."""
    return DirectoryValidator(directory, name).check_exists().check_not_symlink().validate()


def file_safe_check(name: str, path: Any, unsupported_mode: int = 0o022, min_size: int = 1, max_size: int = 1 << 40) -> str:
    """An existing regular file that may be trusted as input: not a symbolic link, size within ``[min_size, max_size]``, none
    of the ``unsupported_mode`` permission bits set (default: not writable by group / others), owned by the caller or root."""
    v = StringValidator(path, name, 4096)
    v.add(lambda p: os.path.isfile(p) and not os.path.islink(p), "must be an existing regular file, not a symbolic link")
    v.add(lambda p: min_size <= os.path.getsize(p) <= max_size, "size must be in [%d, %d] bytes" % (min_size, max_size))
    v.add(lambda p: (os.stat(p).st_mode & unsupported_mode) == 0, "must not have permission bits %o" % unsupported_mode)
    v.add(lambda p: os.stat(p).st_uid in (os.getuid(), 0), "must be owned by the calling user or root")
    return v.validate()


def path_safe_check(name: str, value: Any, must_exist: bool = False) -> str:
    v = DirectoryValidator(value, name).check_not_symlink()
    if must_exist:
        v.check_exists()
    return v.validate()


# ----------------------------------------------------------------------------------------------------------------------
# Typed validators and the decorator form (reference: validator.py:99-196 para_checker_decorator, :199-330 Class / List /
# Or / And / Option validators, :482-620 numeric validators, :720-780 FileValidator)
# ----------------------------------------------------------------------------------------------------------------------
class NumValidator(Validator):
    """Number in a closed, open or half-open interval; ``bool`` is never a number here."""

    def __init__(self, value: Any, name: str = "value", min_value=None, max_value=None, interval: str = "[]") -> None:
        super().__init__(value, name)
        if interval not in ("[]", "()", "(]", "[)"):
            raise ValueError("interval must be one of [] () (] [)")
        self.check_type(int, float)
        lo_open, hi_open = interval[0] == "(", interval[1] == ")"
        self.add(lambda v: (min_value is None or (v > min_value if lo_open else v >= min_value))
                 and (max_value is None or (v < max_value if hi_open else v <= max_value)),
                 "must be in %s%s, %s%s" % (interval[0], min_value, max_value, interval[1]))


class IntValidator(NumValidator):
    def __init__(self, value: Any, name: str = "value", min_value: Optional[int] = None, max_value: Optional[int] = None,
                 interval: str = "[]") -> None:
        super().__init__(value, name, min_value, max_value, interval)
        self._checks.insert(0, (lambda v: isinstance(v, int) and not isinstance(v, bool), "must be an int"))


class FloatValidator(NumValidator):
    def __init__(self, value: Any, name: str = "value", min_value: Optional[float] = None, max_value: Optional[float] = None,
                 interval: str = "[]") -> None:
        super().__init__(value, name, min_value, max_value, interval)
        self._checks.insert(0, (lambda v: isinstance(v, float), "must be a float"))


class Convert2intValidator(IntValidator):
    """A string (or number) that converts to an int inside the range; ``validate`` returns the int."""

    def __init__(self, value: Any, name: str = "value", min_value: Optional[int] = None, max_value: Optional[int] = None) -> None:
        try:
            conv = int(value) if not isinstance(value, bool) else value
        except (TypeError, ValueError):
            conv = value
        super().__init__(conv, name, min_value, max_value)


class _Optional:
    """Mixin: ``None`` passes."""

    def validate(self):  # type: ignore[override]
        return None if self.value is None else super().validate()  # type: ignore[misc]


class OptionalIntValidator(_Optional, IntValidator):
    pass


class OptionalFloatValidator(_Optional, FloatValidator):
    pass


class OptionalStringValidator(_Optional, StringValidator):
    pass


class ClassValidator(Validator):
    def __init__(self, value: Any, name: str = "value", classes=()) -> None:
        super().__init__(value, name)
        classes = tuple(classes) if isinstance(classes, (list, tuple)) else (classes,)
        self.add(lambda v: isinstance(v, classes), "must be an instance of %s" % "/".join(c.__name__ for c in classes))


class OptionValidator(Validator):
    def __init__(self, value: Any, name: str = "value", options: Iterable = ()) -> None:
        super().__init__(value, name)
        self.check_in(options)


class ListValidator(Validator):
    """Every element passes ``sub_validator(element, name[i], **kwargs)``; optional length bounds."""

    def __init__(self, value: Any, name: str = "value", sub_validator: type = Validator, min_len: int = 0,
                 max_len: Optional[int] = None, **kwargs) -> None:
        super().__init__(value, name)
        self.check_type(list, tuple).check_length(min_len, max_len)

        def all_ok(v):
            for i, x in enumerate(v):
                sub_validator(x, "%s[%d]" % (name, i), **kwargs).validate()
            return True

        self.add(all_ok, "has an invalid element")


class OrValidator(Validator):
    """Passes when at least one of the given validators passes."""

    def __init__(self, value: Any, name: str = "value", options: Iterable[Validator] = ()) -> None:
        super().__init__(value, name)
        opts = list(options)
        self.add(lambda _v: any(o.is_valid() for o in opts), "matches none of the accepted forms")


class AndValidator(Validator):
    def __init__(self, value: Any, name: str = "value", options: Iterable[Validator] = ()) -> None:
        super().__init__(value, name)
        opts = list(options)
        self.add(lambda _v: all(o.is_valid() for o in opts), "fails one of the required checks")


class FileValidator(StringValidator):
    """An existing regular file that may be trusted as input: bounded size, not a symbolic link, owned by the caller (or
    root), not writable by group / others."""

    def __init__(self, value: Any, name: str = "file", max_len: int = 1024) -> None:
        super().__init__(value, name, max_len)
        self.add(lambda v: ".." not in v.replace("\\", "/").split("/"), "must not contain '..'")

    def check_not_soft_link(self) -> "FileValidator":
        return self.add(lambda v: not os.path.islink(v), "must not be a symbolic link")  # type: ignore[return-value]

    def check_file_size(self, max_size: int = 1 << 40, min_size: int = 0) -> "FileValidator":
        return self.add(lambda v: os.path.isfile(v) and min_size <= os.path.getsize(v) <= max_size,
                        "must be a file of %d..%d bytes" % (min_size, max_size))  # type: ignore[return-value]

    def check_user_group(self) -> "FileValidator":
        return self.add(lambda v: os.stat(v).st_uid in (os.geteuid(), 0), "must be owned by the calling user or root")  # type: ignore[return-value]

    def check_file_mode(self, unsupported_mode: int = 0o022) -> "FileValidator":
        return self.add(lambda v: (os.stat(v).st_mode & unsupported_mode) == 0,
                        "must not be writable by group or others")  # type: ignore[return-value]


def para_checker_decorator(check_option_list: List[tuple]):
    """``@para_checker_decorator([("lr", FloatValidator, {"min_value": 0.0}), (["a", "b"], ClassValidator, {"classes": int})])``
    validates the named arguments of the decorated function (positional or keyword, defaults included) before the call.
    Each option is ``(name or list of names, validator class, constructor keywords[, list of chain methods to call])``."""
    import functools
    import inspect

    def deco(func):
        sig = inspect.signature(func)

        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            bound = sig.bind(*args, **kwargs)
            bound.apply_defaults()
            for opt in check_option_list:
                names, cls = opt[0], opt[1]
                kw = dict(opt[2]) if len(opt) > 2 and opt[2] else {}
                chain = list(opt[3]) if len(opt) > 3 and opt[3] else []
                for n in (names if isinstance(names, (list, tuple)) else [names]):
                    if n not in bound.arguments:
                        raise ValidationError("%s() has no argument %r to validate" % (func.__name__, n))
                    v = cls(bound.arguments[n], n, **kw)
                    for m in chain:
                        getattr(v, m)()
                    v.validate()
            return func(*args, **kwargs)

        return wrapper

    return deco
