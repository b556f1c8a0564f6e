"""LibraryTaskDescriptor and Access, as in the reference
(tornado-api/.../common/LibraryTaskDescriptor.java:30-91, common/Access.java)."""
from __future__ import annotations

import enum
from typing import Any, Sequence


class Access(enum.Enum):
    READ_ONLY = 1
    WRITE_ONLY = 2
    READ_WRITE = 3


class LibraryTaskDescriptor:
    def __init__(self):
        self._library = None
        self._function = None
        self._parameters: Sequence[Any] = ()
        self._access: Sequence[Access] = ()
        self._tuning = None

    def withLibrary(self, name):  # noqa: N802
        self._library = name
        return self

    def withFunction(self, name):  # noqa: N802
        self._function = name
        return self

    def withParameters(self, params):  # noqa: N802
        self._parameters = list(params)
        return self

    def withAccess(self, access):  # noqa: N802
        self._access = list(access)
        return self

    def withTuning(self, tuning):  # noqa: N802
        self._tuning = tuning
        return self

    def getLibraryName(self):  # noqa: N802
        return self._library

    def getFunctionName(self):  # noqa: N802
        return self._function

    def getParameters(self):  # noqa: N802
        return self._parameters

    def getAccess(self):  # noqa: N802
        return self._access

    def getTuning(self):  # noqa: N802
        return self._tuning
