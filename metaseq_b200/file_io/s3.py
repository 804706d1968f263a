"""``s3://<bucket>/<key>`` behind the path manager.

Reading downloads the object into a local cache (refreshed when the object is newer than the cached file) and
opens that file; writing collects into a memory buffer that is uploaded as one object when the handle is closed.
Directories are key prefixes: ``ls`` lists one level, ``mkdirs`` writes the empty ``<prefix>/`` marker object.
``boto3`` is imported on first use; a ``client_factory`` can be given instead, which is how the tests drive the
handler against an in-memory bucket.  Reference: metaseq/file_io/s3.py.
"""
from __future__ import annotations

import datetime
import io
import logging
import os
import shutil
from typing import Any, Callable, Dict, List, Optional, Tuple

from .path_manager import PathHandler

logger = logging.getLogger(__name__)


def _is_client_error(exc: BaseException) -> bool:
    return type(exc).__name__ in ("ClientError", "NoCredentialsError", "EndpointConnectionError")


def s3_close_and_upload(buffer, client, bucket: str, s3_path: str, transfer_config=None) -> None:
    """Uploads what was written to ``buffer`` (a ``BytesIO`` or ``StringIO``) as one object, then really closes it."""
    body = buffer.getvalue()
    if isinstance(body, str):
        body = body.encode("utf-8")
    extra = {"Config": transfer_config} if transfer_config is not None else {}
    try:
        client.upload_fileobj(io.BytesIO(body), bucket, s3_path, **extra)
    except Exception as e:  # noqa: BLE001
        if _is_client_error(e):
            raise OSError(f"Error in file upload - {type(e).__name__}: {e}") from e
        raise
    finally:
        type(buffer).close(buffer)


class S3PathHandler(PathHandler):
    S3_PREFIX = "s3://"
    CACHE_SUBDIR_NAME = "s3_cache"

    def __init__(self, cache_dir: Optional[str] = None, transfer_config_kwargs: Optional[Dict] = None,
                 client_factory: Optional[Callable[[], Any]] = None):
        """``transfer_config_kwargs`` go to ``boto3.s3.transfer.TransferConfig`` (multipart thresholds, concurrency).
        ``client_factory()`` returns the client to use instead of ``boto3.client("s3")``."""
        self.cache_dir = cache_dir
        self._transfer_kwargs = transfer_config_kwargs or {}
        self._client_factory = client_factory
        self.client = None
        self._transfer_config = None

    def _get_supported_prefixes(self) -> List[str]:
        return [self.S3_PREFIX]

    def _parse_uri(self, uri: str) -> Tuple[str, str]:
        """``s3://<bucket>/<key>`` -> ``(bucket, key)``."""
        rest = uri[len(self.S3_PREFIX):] if uri.startswith(self.S3_PREFIX) else None
        if not rest or "/" not in rest:
            raise ValueError(f"Expected s3://<bucket>/<path>: {uri}")
        bucket, _, key = rest.partition("/")
        return bucket, key

    def _get_client(self, bucket: str):
        if self.client is None:
            if self._client_factory is not None:
                self.client = self._client_factory()
            else:
                try:
                    import boto3
                    from boto3.s3.transfer import TransferConfig
                except ImportError as e:
                    raise ImportError("s3:// paths need the boto3 package (pip install boto3)") from e
                try:
                    self.client = boto3.client("s3")
                except Exception as e:  # noqa: BLE001
                    raise OSError(f"Error in making s3 client for bucket {bucket}: {type(e).__name__}: {e}") from e
                self._transfer_config = TransferConfig(**self._transfer_kwargs)
        return self.client

    @property
    def transfer_config(self):
        return self._transfer_config

    def _config_args(self) -> Dict[str, Any]:
        return {"Config": self._transfer_config} if self._transfer_config is not None else {}

    # ----------------------------------------------------------------- queries
    def _head_object(self, path: str) -> Optional[Dict]:
        bucket, key = self._parse_uri(path)
        try:
            return self._get_client(bucket).head_object(Bucket=bucket, Key=key)
        except Exception as e:  # noqa: BLE001
            code = getattr(e, "response", {}).get("Error", {}).get("Message", "")
            if _is_client_error(e) and code == "Bad Request":
                raise OSError(f"Error in checking s3 path {path} - {type(e).__name__}: {e}") from e
            if _is_client_error(e) or isinstance(e, KeyError):
                return None
            raise

    def _isfile(self, path: str, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        return not path.endswith("/") and self._head_object(path) is not None

    def _isdir(self, path: str, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        bucket, key = self._parse_uri(path)
        prefix = key if key.endswith("/") or not key else key + "/"
        resp = self._get_client(bucket).list_objects_v2(Bucket=bucket, Prefix=prefix, MaxKeys=1)
        return resp.get("KeyCount", len(resp.get("Contents", []))) > 0

    def _exists(self, path: str, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        return self._isfile(path) or self._isdir(path)

    def _ls(self, path: str, **kwargs) -> List[str]:
        """Full keys of the objects, and prefixes of the sub-directories, one level below ``path``."""
        self._check_kwargs(kwargs)
        bucket, key = self._parse_uri(path)
        prefix = key if key.endswith("/") or not key else key + "/"
        client = self._get_client(bucket)
        out: List[str] = []
        token = None
        while True:
            args = dict(Bucket=bucket, Prefix=prefix, Delimiter="/")
            if token:
                args["ContinuationToken"] = token
            resp = client.list_objects_v2(**args)
            out += [o["Key"] for o in resp.get("Contents", []) if o["Key"] != prefix]
            out += [p["Prefix"] for p in resp.get("CommonPrefixes", [])]
            if not resp.get("IsTruncated"):
                return out
            token = resp.get("NextContinuationToken")

    # ------------------------------------------------------------- local cache
    def _local_cache_path(self, path: str) -> str:
        from . import get_cache_dir

        _, key = self._parse_uri(path)
        return os.path.join(get_cache_dir(self.cache_dir), self.CACHE_SUBDIR_NAME, key)

    def _get_local_path(self, path: str, force: bool = False, **kwargs) -> str:
        """A cached local copy of the object; downloaded again when the object is newer than the copy or with
        ``force``."""
        self._check_kwargs(kwargs)
        if path.endswith("/"):
            raise NotImplementedError("S3PathHandler does not currently support downloading directories")
        assert self._isfile(path), f"File not found: {path}"
        from . import file_lock

        local = self._local_cache_path(path)
        with file_lock(local):
            if os.path.exists(local) and not force:
                head = self._head_object(path)
                if head is not None:
                    remote = head["LastModified"].astimezone(datetime.timezone.utc)
                    mine = datetime.datetime.fromtimestamp(os.path.getmtime(local), tz=datetime.timezone.utc)
                    if mine > remote:
                        logger.info("URL {} was already cached in {}".format(path, local))
                        return local
            logger.info("Caching {} ...".format(path))
            os.makedirs(os.path.dirname(local) or ".", exist_ok=True)
            tmp = local + ".tmp"
            if os.path.isfile(tmp):
                os.unlink(tmp)  # left behind by a process that died mid-download
            bucket, key = self._parse_uri(path)
            try:
                self._get_client(bucket).download_file(bucket, key, tmp, **self._config_args())
                shutil.move(tmp, local)  # a rename: readers never see a partial file
            finally:
                if os.path.exists(tmp):
                    os.unlink(tmp)
            logger.info("URL {} cached in {}".format(path, local))
        return local

    # -------------------------------------------------------------------- I/O
    def _open(self, path: str, mode: str = "r", buffering: int = -1, encoding: Optional[str] = None,
              errors: Optional[str] = None, newline: Optional[str] = None, read_chunk_size: Optional[int] = None,
              **kwargs):
        self._check_kwargs(kwargs)
        bucket, key = self._parse_uri(path)
        base = mode.replace("b", "").replace("t", "")
        if base == "r":
            local = self._get_local_path(path)
            if "b" in mode:
                return open(local, mode, buffering=buffering)
            return open(local, mode, buffering=buffering, encoding=encoding, errors=errors, newline=newline)
        if base != "w":
            raise OSError(f"Unsupported open mode {mode}")
        client = self._get_client(bucket)
        buffer: Any = io.BytesIO() if "b" in mode else io.StringIO()
        handler = self

        def close():
            if not buffer.closed:
                s3_close_and_upload(buffer, client, bucket, key, handler._transfer_config)

        buffer.close = close
        return buffer

    def _copy_from_local(self, local_path: str, dst_path: str, overwrite: bool = False, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        if dst_path.endswith("/"):
            raise NotImplementedError("S3PathHandler does not currently support uploading directories")
        if not overwrite and self._isfile(dst_path):
            logger.error(f"Error: Destination path {dst_path} already exists.")
            return False
        bucket, key = self._parse_uri(dst_path)
        try:
            self._get_client(bucket).upload_file(local_path, bucket, key, **self._config_args())
            return True
        except Exception as e:  # noqa: BLE001
            if _is_client_error(e):
                logger.error(f"Error in file upload - {e}")
                return False
            raise

    def _copy(self, src_path: str, dst_path: str, overwrite: bool = False, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        src_bucket, src_key = self._parse_uri(src_path)
        dst_bucket, dst_key = self._parse_uri(dst_path)
        assert src_bucket == dst_bucket, "For now, can only _copy() within a bucket."
        if not overwrite and self._isfile(dst_path):
            logger.error(f"Error: Destination path {dst_path} already exists.")
            return False
        try:
            self._get_client(src_bucket).copy({"Bucket": src_bucket, "Key": src_key}, dst_bucket, dst_key,
                                              **self._config_args())
            return True
        except Exception as e:  # noqa: BLE001
            if _is_client_error(e):
                logger.error(f"Error in file copy - {e}")
                return False
            raise

    def _mkdirs(self, path: str, **kwargs) -> None:
        self._check_kwargs(kwargs)
        assert path.endswith("/"), path
        bucket, key = self._parse_uri(path)
        try:
            self._get_client(bucket).put_object(Bucket=bucket, Key=key)
        except Exception as e:  # noqa: BLE001
            raise OSError(f"Error in mkdirs path {path} - {type(e).__name__}: {e}") from e

    def _rm(self, path: str, **kwargs) -> None:
        self._check_kwargs(kwargs)
        bucket, key = self._parse_uri(path)
        try:
            self._get_client(bucket).delete_object(Bucket=bucket, Key=key)
        except Exception as e:  # noqa: BLE001
            raise OSError(f"Error in rm path {path} - {type(e).__name__}: {e}") from e

    def _close(self):
        self.client = None
