"""Container deployment: entry point that maps a memory profile onto ``serve`` flags, and a host-side launcher that
builds the ``docker run`` command line (reference: scripts/agens-entry.sh, scripts/agens-run.sh,
docker/Dockerfile.release)."""
