"""Azure Blob Storage behind the path manager: ``az://<account>/<container>/<blob path>`` (or ``blob://``).

Reads stream the blob chunk by chunk (``AzureBlobReader``); writes stage fixed-size blocks and commit the block
list on close (``AzureBlobWriter``), so neither side holds a whole checkpoint in memory.  Authentication is a SAS
token from a ``AzureBlobTokenProvider`` (by default the ``AZURE_STORAGE_SAS_TOKEN`` environment variable).
``get_local_path`` keeps a local cache that is refreshed when the blob is newer than the cached file.

The SDK (``azure-storage-blob``) is imported on first use; a ``service_factory`` can be given instead, which is
how the tests drive the handler against an in-memory service.  Reference: metaseq/file_io/azure_blob.py.
"""
from __future__ import annotations

import base64
import datetime
import io
import logging
import os
import shutil
import time
from types import SimpleNamespace
from typing import Any, Callable, Dict, List, Optional, Tuple

from .path_manager import PathHandler

logger = logging.getLogger(__name__)

DEFAULT_CHUNK_SIZE = 4 * 1024 * 1024
ENV_SAS_TOKEN = "AZURE_STORAGE_SAS_TOKEN"


def _sdk():
    try:
        import azure.storage.blob as azure_blob
    except ImportError as e:
        raise ImportError("az:// paths need the azure-storage-blob package (pip install azure-storage-blob)") from e
    return azure_blob


def _is_not_found(exc: BaseException) -> bool:
    return type(exc).__name__ == "ResourceNotFoundError"


class AzureBlobTokenProvider:
    def get_sas_token(self, account: str) -> str:
        """A SAS token for the storage account."""
        raise NotImplementedError


class EnvironmentTokenProvider(AzureBlobTokenProvider):
    def get_sas_token(self, _: str) -> str:
        assert ENV_SAS_TOKEN in os.environ, f"Missing required env variable: {ENV_SAS_TOKEN}"
        return os.environ[ENV_SAS_TOKEN]


class _Unsupported:
    """The file-object calls that a one-directional stream refuses."""

    def seekable(self):
        return False

    def seek(self, offset: int, whence: int = os.SEEK_SET) -> int:
        raise io.UnsupportedOperation()

    def tell(self):
        raise io.UnsupportedOperation()

    def truncate(self, size=None):
        raise io.UnsupportedOperation()


class AzureBlobReader(_Unsupported, io.RawIOBase):
    """Read-only stream over a blob client: one ranged download of ``chunk_size`` bytes at a time, sliced out to
    the caller until it is used up."""

    def __init__(self, client, chunk_size: int = DEFAULT_CHUNK_SIZE):
        super().__init__()
        self._client = client
        self._chunks = client.download_blob().chunks()
        self._chunk_size = chunk_size
        self._chunk: Optional[bytes] = None
        self._pos = 0

    def _take(self, size: int) -> bytes:
        """Up to ``size`` bytes of the current chunk (fetching the next one when it is exhausted); empty at EOF."""
        if size == 0:
            return b""
        if self._chunk is None or self._pos >= len(self._chunk):
            try:
                self._chunk = next(self._chunks)
            except StopIteration:
                return b""
            self._pos = 0
            logger.info("Read next chunk: blob_name=%s, length=%d", self._client.blob_name, len(self._chunk))
        data = self._chunk[self._pos:self._pos + size]
        self._pos += len(data)
        return data

    def readable(self):
        return True

    def writable(self):
        return False

    writeable = writable  # the reference's spelling

    def read(self, size: int = -1) -> bytes:
        return self.readall() if size is None or size < 0 else self._take(size)

    def readall(self) -> bytes:
        out = io.BytesIO()
        self.readinto(out)
        return out.getvalue()

    def readinto(self, stream):
        """Copies the rest of the blob into ``stream`` (anything with ``write``); a buffer is filled as for any
        raw stream."""
        if not hasattr(stream, "write"):
            data = self._take(len(stream))
            stream[:len(data)] = data
            return len(data)
        data = self._take(self._chunk_size)
        while data:
            stream.write(data)
            data = self._take(self._chunk_size)

    def write(self, b):
        raise io.UnsupportedOperation()


class AzureBlobWriter(_Unsupported, io.RawIOBase):
    """Write-only stream: data collects in a buffer of ``chunk_size`` bytes; each full buffer (and ``flush``) is
    staged as one block with a fixed-width id, and ``close`` commits the block list, which makes the blob appear."""

    MAX_BLOCKS = 50000

    def __init__(self, client, chunk_size: int = DEFAULT_CHUNK_SIZE, block_factory: Optional[Callable] = None):
        super().__init__()
        self._client = client
        self._chunk_size = chunk_size
        self._buffer: Optional[io.BytesIO] = None
        self._blocks: List[Any] = []
        self._make_block = block_factory
        self._finished = False

    def _block_id(self, index: int) -> str:
        # ids must be base64, of one length for all blocks of a blob
        assert index < self.MAX_BLOCKS, "a block blob holds at most 50000 blocks: raise the chunk size"
        return base64.urlsafe_b64encode("{0:05}".format(index).encode("utf-8")).decode("utf-8")

    def readable(self):
        return False

    def writable(self):
        return True

    writeable = writable

    def read(self, size: int = -1):
        raise io.UnsupportedOperation()

    def write(self, b) -> int:
        if self._buffer is None or self._buffer.tell() >= self._chunk_size:
            self.flush()
            self._buffer = io.BytesIO()
        return self._buffer.write(b)

    def flush(self):
        if self._buffer is None or self._buffer.tell() == 0:
            return
        block_id = self._block_id(len(self._blocks))
        length = self._buffer.tell()
        self._buffer.seek(0)
        logger.info("Uploading a new block: blob_name=%s, block_id=%s, idx=%d, length=%d", self._client.blob_name,
                    block_id, len(self._blocks), length)
        self._client.stage_block(block_id, self._buffer, length)
        if self._make_block is None:
            self._make_block = lambda block_id: _sdk().BlobBlock(block_id=block_id)
        self._blocks.append(self._make_block(block_id))
        self._buffer = None

    def close(self):
        if self._finished:
            return
        self._finished = True
        self.flush()
        if self._blocks:
            logger.info("Committing blocks: blob_name=%s, count=%d", self._client.blob_name, len(self._blocks))
            self._client.commit_block_list(self._blocks)
        super().close()

    def __exit__(self, *exc):
        self.close()  # commit even when the body raised: what was written stays readable


class AzureBlobPathHandler(PathHandler):
    SUPPORTED_PREFIXES = ["az://", "blob://"]
    CACHE_SUBDIR_NAME = "blob_cache"

    def __init__(self, token_provider: Optional[AzureBlobTokenProvider] = None, cache_dir: Optional[str] = None,
                 service_factory: Optional[Callable[[str, str], Any]] = None, block_factory: Optional[Callable] = None):
        """``service_factory(account_url, sas_token)`` returns the service client (default: the SDK's
        ``BlobServiceClient``); ``block_factory(block_id)`` the entries of a block list (default: ``BlobBlock``)."""
        self.token_provider = token_provider or EnvironmentTokenProvider()
        self.cache_dir = cache_dir
        self._service_factory = service_factory
        self._block_factory = block_factory
        self._clients: Dict[str, Any] = {}

    def _get_supported_prefixes(self) -> List[str]:
        return self.SUPPORTED_PREFIXES

    # ------------------------------------------------------------------ naming
    def _parse_uri(self, uri: str) -> Tuple[str, str, str]:
        """``az://<account>/<container>/<path>`` -> ``(account, container, path)``."""
        for prefix in self.SUPPORTED_PREFIXES:
            if uri.startswith(prefix):
                parts = uri[len(prefix):].split("/")
                if len(parts) < 2 or not parts[0] or not parts[1]:
                    raise ValueError(f"Expected {prefix}<account>/<container>/<path>: {uri}")
                return parts[0], parts[1], "/".join(parts[2:])
        raise ValueError(f"Unsupported URI: {uri}")

    def _get_service_uri(self, account: str, container: str, blob_path: str, include_auth: bool = False) -> str:
        uri = "/".join(p for p in (f"https://{account}.blob.core.windows.net", container, blob_path) if p)
        if include_auth:
            uri += "?" + self.token_provider.get_sas_token(account)
        return uri

    def _get_client(self, account: str):
        if account not in self._clients:
            url = f"https://{account}.blob.core.windows.net"
            token = self.token_provider.get_sas_token(account)
            factory = self._service_factory or (lambda u, t: _sdk().BlobServiceClient(u, credential=t))
            self._clients[account] = factory(url, token)
        return self._clients[account]

    def _blob_client(self, path: str):
        account, container, blob = self._parse_uri(path)
        return self._get_client(account).get_blob_client(container=container, blob=blob)

    def _get_blob_properties(self, path: str) -> Optional[Dict]:
        return dict(self._blob_client(path).get_blob_properties().items())

    def _enumerate_blobs(self, path: str):
        account, container, blob = self._parse_uri(path)
        return self._get_client(account).get_container_client(container).list_blobs(name_starts_with=blob)

    # ----------------------------------------------------------------- queries
    def _isfile(self, path: str, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        if path.endswith("/"):
            return False
        try:
            return self._get_blob_properties(path) is not None
        except Exception as e:  # noqa: BLE001
            if _is_not_found(e):
                return False
            logger.error(f"Error in isfile - {e}")
            return False

    def _isdir(self, path: str, **kwargs) -> bool:
        """There are no directories in blob storage: a path is one if some blob's name continues it after a
        slash."""
        self._check_kwargs(kwargs)
        prefix = path if path.endswith("/") else path + "/"
        _, _, dir_name = self._parse_uri(prefix)
        try:
            first = next(iter(self._enumerate_blobs(prefix)), None)
            return first is not None and len(first.name) > len(dir_name)
        except Exception as e:  # noqa: BLE001
            if not _is_not_found(e):
                logger.error(f"Error in isdir - {e}")
            return False

    def _exists(self, path: str, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        return self._isfile(path) or self._isdir(path)

    def _ls(self, path: str, **kwargs) -> List[str]:
        """Names (from the container root) of every blob under ``path``."""
        self._check_kwargs(kwargs)
        return [b.name for b in self._enumerate_blobs(path)]

    # ------------------------------------------------------------- local cache
    def _local_cache_path(self, path: str) -> str:
        from . import get_cache_dir

        _, _, blob = self._parse_uri(path)
        return os.path.join(get_cache_dir(self.cache_dir), self.CACHE_SUBDIR_NAME, blob)

    def _get_local_path(self, path: str, force: bool = False, **kwargs) -> str:
        """A local copy of a blob, or of every blob under a directory path.  A cached file is reused unless the
        blob was modified after it was written (or ``force``)."""
        self._check_kwargs(kwargs)
        assert self._exists(path), f"File not found: {path}"
        result = self._local_cache_path(path)
        if self._isdir(path):
            account, container, _ = self._parse_uri(path)
            for name in self._ls(path):
                self._get_local_path_single(f"az://{account}/{container}/{name}", force=force)
        else:
            self._get_local_path_single(path, force=force)
        return result

    def _get_local_path_single(self, path: str, force: bool = False) -> str:
        from . import file_lock

        local = self._local_cache_path(path)
        with file_lock(local):
            if os.path.exists(local) and not force:
                remote_time = self._get_blob_properties(path).get("last_modified")
                local_time = datetime.datetime.fromtimestamp(os.path.getmtime(local), tz=datetime.timezone.utc)
                if remote_time is None or remote_time.astimezone(datetime.timezone.utc) <= local_time:
                    logger.info("URL {} was already cached in {}".format(path, local))
                    return local
                logger.info("Remote file {} is newer than the cached one: downloading again".format(path))
            os.makedirs(os.path.dirname(local) or ".", exist_ok=True)
            tmp = local + ".tmp"
            with open(tmp, "wb") as out:
                self._blob_client(path).download_blob().readinto(out)
            shutil.move(tmp, local)
            logger.info("URL {} cached in {}".format(path, local))
        return local

    # -------------------------------------------------------------------- I/O
    def _open(self, path: str, mode: str = "rb", buffering: int = -1, encoding: Optional[str] = None,
              errors: Optional[str] = None, newline: Optional[str] = None, **kwargs):
        """``rb`` -> streaming reader, ``wb`` -> block writer; ``buffering`` > 0 sets the chunk size.  Text modes
        wrap the same streams."""
        self._check_kwargs(kwargs)
        chunk = buffering if buffering and buffering > 0 else DEFAULT_CHUNK_SIZE
        text = "b" not in mode
        base = mode.replace("b", "").replace("t", "")
        if base == "r":
            raw: Any = io.BufferedReader(AzureBlobReader(self._blob_client(path), chunk), buffer_size=min(chunk, 1 << 20))
        elif base == "w":
            raw = AzureBlobWriter(self._blob_client(path), chunk, self._block_factory)
        else:
            raise ValueError(f"Supported modes: rb, wb (and their text forms), not {mode}")
        if not text:
            return raw
        return io.TextIOWrapper(raw if base == "r" else io.BufferedWriter(raw, buffer_size=min(chunk, 1 << 20)),
                                encoding=encoding or "utf-8", errors=errors, newline=newline)

    def _mkdirs(self, path: str, **kwargs) -> None:
        self._check_kwargs(kwargs)  # nothing to make: directories exist through their blobs

    def _copy_from_local(self, local_path: str, dst_path: str, overwrite: bool = False, **kwargs) -> bool:
        self._check_kwargs(kwargs)
        if os.path.isdir(local_path):
            raise NotImplementedError("AzureBlobPathHandler does not currently support uploading directories")
        if not overwrite and self._isfile(dst_path):
            logger.error(f"Error: Destination path {dst_path} already exists.")
            return False
        try:
            with open(local_path, "rb") as src:
                self._blob_client(dst_path).upload_blob(src, length=os.path.getsize(local_path), overwrite=overwrite)
            return True
        except Exception as e:  # noqa: BLE001
            logger.error(f"Error in file upload - {e}")
            return False

    def _copy(self, src_path: str, dst_path: str, overwrite: bool = False, **kwargs) -> bool:
        """Server-side copy between two blobs; waits for it to finish."""
        self._check_kwargs(kwargs)
        if not overwrite and self._isfile(dst_path):
            logger.error(f"Error: Destination path {dst_path} already exists.")
            return False
        try:
            source = self._get_service_uri(*self._parse_uri(src_path), include_auth=True)
            dst = self._blob_client(dst_path)
            dst.start_copy_from_url(source)
            return self._wait_for_copy(dst)
        except Exception as e:  # noqa: BLE001
            logger.error(f"Error in blob copy - {e}")
            return False

    @staticmethod
    def _wait_for_copy(blob_client, attempts: int = 20, sleep_seconds: float = 3.0) -> bool:
        for _ in range(attempts):
            status = blob_client.get_blob_properties().copy.status
            if status != "pending":
                return status == "success"
            time.sleep(sleep_seconds)
        return False

    def _rm(self, path: str, **kwargs) -> None:
        self._check_kwargs(kwargs)
        try:
            self._blob_client(path).delete_blob()
        except Exception as e:  # noqa: BLE001
            raise OSError(f"Error in rm path {path} - {type(e).__name__}: {e}") from e

    def _close(self):
        for client in self._clients.values():
            close = getattr(client, "close", None)
            if close is not None:
                close()
        self._clients = {}


def blob_block(block_id: str):
    """A block-list entry without the SDK (``block_factory`` of a handler that talks to a stand-in service)."""
    return SimpleNamespace(id=block_id)
