"""Local cache for model archives and vocabulary files referenced by URL or path
(reference: metaseq/file_utils.py).  There is no network access in many deployments, so every remote
fetch is attempted only when the file is not already cached and fails with a clear error otherwise."""
from __future__ import annotations

import fnmatch
import functools
import json
import logging
import os
import shutil
import tarfile
import tempfile
from hashlib import sha256
from urllib.parse import urlparse

logger = logging.getLogger(__name__)

try:
    from torch.hub import _get_torch_home

    _default_cache = os.path.join(_get_torch_home(), "pytorch_fairseq")
except Exception:  # noqa: BLE001
    _default_cache = os.path.expanduser(os.path.join("~", ".cache", "torch", "pytorch_fairseq"))
PYTORCH_FAIRSEQ_CACHE = os.getenv("PYTORCH_FAIRSEQ_CACHE", _default_cache)

CONFIG_NAME = "config.json"
WEIGHTS_NAME = "pytorch_model.bin"


def url_to_filename(url, etag=None):
    """Cache file name: hash of the URL, plus ``.<hash of the ETag>`` when one is known."""
    name = sha256(url.encode("utf-8")).hexdigest()
    if etag:
        name += "." + sha256(etag.encode("utf-8")).hexdigest()
    return name


def split_s3_path(url):
    parsed = urlparse(url)
    if not parsed.netloc or not parsed.path:
        raise ValueError("bad s3 path {}".format(url))
    return parsed.netloc, parsed.path.lstrip("/")


def s3_request(func):
    """Decorator for S3 calls: a missing object becomes ``EnvironmentError("file ... not found")``."""

    @functools.wraps(func)
    def wrapper(url, *args, **kwargs):
        from botocore.exceptions import ClientError

        try:
            return func(url, *args, **kwargs)
        except ClientError as exc:
            if str(exc.response.get("Error", {}).get("Code")) == "404":
                raise EnvironmentError("file {} not found".format(url)) from exc
            raise

    return wrapper


@s3_request
def s3_etag(url):
    import boto3

    bucket, key = split_s3_path(url)
    return boto3.resource("s3").Object(bucket, key).e_tag


@s3_request
def s3_get(url, temp_file):
    import boto3

    bucket, key = split_s3_path(url)
    boto3.resource("s3").Bucket(bucket).download_fileobj(key, temp_file)


_TIMEOUTS = (10, 20, 40, 60, 60)


def request_wrap_timeout(func, url):
    """Calls ``func(timeout=...)`` with growing timeouts until one attempt does not time out."""
    import requests

    for attempt, timeout in enumerate(_TIMEOUTS):
        try:
            return func(timeout=timeout)
        except requests.exceptions.Timeout:
            logger.warning("Request for %s timed-out (attempt %d). Retrying with a timeout of %d secs", url, attempt,
                           _TIMEOUTS[min(attempt + 1, len(_TIMEOUTS) - 1)])
    raise RuntimeError(f"Unable to fetch file {url}")


def http_get(url, temp_file):
    import requests

    req = request_wrap_timeout(functools.partial(requests.get, url, stream=True), url)
    req.raise_for_status()
    for chunk in req.iter_content(chunk_size=1 << 20):
        if chunk:
            temp_file.write(chunk)


def _fetch(url, out_file):
    (s3_get if urlparse(url).scheme == "s3" else http_get)(url, out_file)


def _etag(url):
    try:
        if urlparse(url).scheme == "s3":
            return s3_etag(url)
        import requests

        r = request_wrap_timeout(functools.partial(requests.head, url, allow_redirects=True), url)
        return r.headers.get("ETag") if r.status_code == 200 else None
    except Exception:  # noqa: BLE001 - offline: fall back to whatever is cached
        return None


def get_from_cache(url, cache_dir=None):
    cache_dir = cache_dir or PYTORCH_FAIRSEQ_CACHE
    os.makedirs(cache_dir, exist_ok=True)
    etag = _etag(url)
    cache_path = os.path.join(cache_dir, url_to_filename(url, etag))
    if not os.path.exists(cache_path) and etag is None:
        candidates = [f for f in fnmatch.filter(os.listdir(cache_dir), url_to_filename(url) + ".*")
                      if not f.endswith(".json")]
        if candidates:
            cache_path = os.path.join(cache_dir, candidates[-1])
    if not os.path.exists(cache_path):
        with tempfile.NamedTemporaryFile() as tmp:
            logger.info("%s not found in cache, downloading to %s", url, tmp.name)
            _fetch(url, tmp)
            tmp.flush()
            tmp.seek(0)
            with open(cache_path, "wb") as out:
                shutil.copyfileobj(tmp, out)
            with open(cache_path + ".json", "w") as meta:
                json.dump({"url": url, "etag": etag}, meta)
    return cache_path


def cached_path(url_or_filename, cache_dir=None):
    """A local path for a URL (downloaded into the cache once) or for an existing local file."""
    url_or_filename = str(url_or_filename)
    scheme = urlparse(url_or_filename).scheme
    if scheme in ("http", "https", "s3"):
        return get_from_cache(url_or_filename, cache_dir)
    if os.path.exists(url_or_filename):
        return url_or_filename
    if scheme == "":
        raise EnvironmentError("file {} not found".format(url_or_filename))
    raise ValueError("unable to parse {} as a URL or as a local path".format(url_or_filename))


def load_archive_file(archive_file):
    """Resolves an archive (a directory, or a tar file that is extracted next to the cache) to a directory."""
    try:
        resolved = cached_path(archive_file)
    except EnvironmentError:
        logger.info("Archive name '%s' was not found in archive name list or as a path / url.", archive_file)
        return None
    if resolved != archive_file:
        logger.info("loading archive file %s from cache at %s", archive_file, resolved)
    if os.path.isdir(resolved):
        return resolved
    target = None
    try:
        target = tempfile.mkdtemp()
        ext = os.path.splitext(archive_file)[1][1:]
        with tarfile.open(resolved, "r:" + ext) as archive:
            top = os.path.commonprefix(archive.getnames())
            archive.extractall(target)  # noqa: S202 - archives come from the operator's own storage
        os.remove(resolved)
        shutil.move(os.path.join(target, top), resolved)
        return resolved
    finally:
        if target is not None:
            shutil.rmtree(target, ignore_errors=True)
