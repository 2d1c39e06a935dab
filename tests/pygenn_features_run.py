"""Runs the reference's own feature tests (tests/features of GeNN 5.4.0, installed beside the PyGeNN build in
oracle/_ref/pygenn_site/ by oracle/Makefile.pygenn) with the B200 backend registered, in this process:

    python tests/pygenn_features_run.py [pytest arguments]

The tests are the reference's, unmodified; `backend` is parametrised over every registered backend, so
`-k b200` selects the plug-in."""
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SITE = os.path.join(REPO, "oracle", "_ref", "pygenn_site")


def main():
    if not os.path.isdir(os.path.join(SITE, "pygenn")):
        print("PyGeNN has not been built (make -f oracle/Makefile.pygenn)")
        return 5
    sys.path.insert(0, SITE)
    sys.path.insert(0, REPO)
    try:
        import bitarray  # noqa: F401  (test_custom_connectivity_update.py imports it)
    except ImportError:
        sys.path.insert(0, os.path.join(REPO, "tests", "standins"))
    os.environ.setdefault("CXX", "/usr/bin/g++")
    os.environ.setdefault("CC", "/usr/bin/gcc")
    os.chdir(os.path.join(SITE, "features"))       # the tests open their .npy fixtures by relative path
    import genn_b200.pygenn_plugin as plugin
    plugin.register()
    import pytest
    return pytest.main(["-p", "no:cacheprovider"] + sys.argv[1:])


if __name__ == "__main__":
    sys.exit(main())
