import sys

from emberserve_b200.cli import main

sys.exit(main())
