"""``s3://bucket/key`` handler on top of boto3 (imported lazily; registration is skipped when
boto3 is not installed).  Reference: metaseq/file_io/s3.py."""
from __future__ import annotations

import io
import logging
import os
import shutil
import tempfile
from typing import List

import boto3  # noqa: F401  (ImportError here disables the handler)

from .path_manager import PathHandler

logger = logging.getLogger(__name__)


class S3PathHandler(PathHandler):
    PREFIX = "s3://"

    def __init__(self, cache_dir=None):
        self.cache_dir = cache_dir
        self._client = None

    def _get_supported_prefixes(self) -> List[str]:
        return [self.PREFIX]

    def _parse(self, uri):
        rest = uri[len(self.PREFIX):]
        bucket, _, key = rest.partition("/")
        return bucket, key

    def client(self):
        if self._client is None:
            self._client = boto3.client("s3")
        return self._client

    def _exists(self, path, **kw):
        b, k = self._parse(path)
        try:
            self.client().head_object(Bucket=b, Key=k)
            return True
        except Exception:
            return self._isdir(path)

    def _isfile(self, path, **kw):
        b, k = self._parse(path)
        try:
            self.client().head_object(Bucket=b, Key=k)
            return True
        except Exception:
            return False

    def _isdir(self, path, **kw):
        b, k = self._parse(path)
        resp = self.client().list_objects_v2(Bucket=b, Prefix=k.rstrip("/") + "/", MaxKeys=1)
        return resp.get("KeyCount", 0) > 0

    def _ls(self, path, **kw):
        b, k = self._parse(path)
        prefix = k.rstrip("/") + "/" if k else ""
        out, token = [], None
        while True:
            args = dict(Bucket=b, Prefix=prefix, Delimiter="/")
            if token:
                args["ContinuationToken"] = token
            resp = self.client().list_objects_v2(**args)
            out += [o["Key"][len(prefix):] for o in resp.get("Contents", [])]
            out += [p["Prefix"][len(prefix):] for p in resp.get("CommonPrefixes", [])]
            if not resp.get("IsTruncated"):
                return out
            token = resp.get("NextContinuationToken")

    def _get_local_path(self, path, **kw):
        b, k = self._parse(path)
        d = self.cache_dir or tempfile.mkdtemp(prefix="s3cache_")
        local = os.path.join(d, k.replace("/", "_"))
        if not os.path.exists(local):
            self.client().download_file(b, k, local)
        return local

    def _open(self, path, mode="r", buffering=-1, **kw):
        if "r" in mode:
            return open(self._get_local_path(path), mode)
        b, k = self._parse(path)
        handler = self

        class _Upload(io.BytesIO):
            def close(self_inner):
                handler.client().put_object(Bucket=b, Key=k, Body=self_inner.getvalue())
                super().close()

        return _Upload()

    def _copy_from_local(self, local_path, dst_path, overwrite=False, **kw):
        b, k = self._parse(dst_path)
        self.client().upload_file(local_path, b, k)
        return True

    def _rm(self, path, **kw):
        b, k = self._parse(path)
        self.client().delete_object(Bucket=b, Key=k)

    def _mkdirs(self, path, **kw):
        pass
