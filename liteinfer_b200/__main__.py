import sys

from liteinfer_b200.cli import main

sys.exit(main())
