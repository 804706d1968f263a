"""``az://`` / ``blob.core.windows.net`` handler on top of azure-storage-blob (registration is
skipped when the SDK is not installed).  Reference: metaseq/file_io/azure_blob.py."""
from __future__ import annotations

import io
import logging
import os
import tempfile
from typing import List
from urllib.parse import urlparse

from azure.storage.blob import BlobServiceClient  # noqa: F401  (ImportError disables the handler)

from .path_manager import PathHandler

logger = logging.getLogger(__name__)


class AzureBlobPathHandler(PathHandler):
    def __init__(self):
        self._svc = None

    def _get_supported_prefixes(self) -> List[str]:
        return ["az://", "https://"]

    def _parse(self, uri):
        u = urlparse(uri)
        if u.scheme == "az":
            container, _, blob = (u.netloc + u.path).partition("/")
            return None, container, blob
        container, _, blob = u.path.lstrip("/").partition("/")
        return f"{u.scheme}://{u.netloc}", container, blob

    def _service(self, account_url):
        if self._svc is None:
            conn = os.environ.get("AZURE_STORAGE_CONNECTION_STRING")
            if conn:
                self._svc = BlobServiceClient.from_connection_string(conn)
            else:
                self._svc = BlobServiceClient(account_url=account_url, credential=os.environ.get("AZURE_STORAGE_SAS"))
        return self._svc

    def _blob(self, path):
        url, container, blob = self._parse(path)
        return self._service(url).get_blob_client(container=container, blob=blob)

    def _exists(self, path, **kw):
        return self._blob(path).exists()

    def _isfile(self, path, **kw):
        return self._exists(path)

    def _isdir(self, path, **kw):
        return len(self._ls(path)) > 0

    def _ls(self, path, **kw):
        url, container, blob = self._parse(path)
        cc = self._service(url).get_container_client(container)
        prefix = blob.rstrip("/") + "/" if blob else ""
        return [b.name[len(prefix):] for b in cc.list_blobs(name_starts_with=prefix)]

    def _get_local_path(self, path, **kw):
        local = os.path.join(tempfile.mkdtemp(prefix="azcache_"), os.path.basename(path))
        with open(local, "wb") as f:
            f.write(self._blob(path).download_blob().readall())
        return local

    def _open(self, path, mode="r", buffering=-1, **kw):
        if "r" in mode:
            return open(self._get_local_path(path), mode)
        blob = self._blob(path)

        class _Upload(io.BytesIO):
            def close(self_inner):
                blob.upload_blob(self_inner.getvalue(), overwrite=True)
                super().close()

        return _Upload()

    def _copy_from_local(self, local_path, dst_path, overwrite=False, **kw):
        with open(local_path, "rb") as f:
            self._blob(dst_path).upload_blob(f, overwrite=overwrite)
        return True

    def _rm(self, path, **kw):
        self._blob(path).delete_blob()

    def _mkdirs(self, path, **kw):
        pass
