"""Where the tests find a checkout of the reference (its golden files and sample models are data for
several tests): ``MIMIR_REFERENCE_DIR`` if set, else a directory named ``reference`` next to this
repository.  Tests skip when neither exists."""
import os


def reference_dir():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("MIMIR_REFERENCE_DIR"), os.path.join(os.path.dirname(here), "reference")):
        if cand and os.path.isdir(cand):
            return cand
    return None
