#!/bin/bash
# SPDX-License-Identifier: Apache-2.0
# Formats the C++ and CUDA sources with clang-format (style file .clang-format at the repository root) and makes
# every such file end with exactly one newline. Counterpart of the reference project's script/format-code.sh.
#   ci/format_code.sh          rewrite the files in place
#   ci/format_code.sh --check  only report files that would change (exit status 1 if any)
set -u
cd "$(dirname "$0")/.."
if ! command -v clang-format >/dev/null 2>&1; then
	echo "clang-format could not be found, please install it."
	exit 2
fi
status=0
while IFS= read -r -d '' file; do
	if [ "${1:-}" = "--check" ]; then
		if ! clang-format --dry-run --Werror "$file" >/dev/null 2>&1 || [ -n "$(tail -c1 "$file")" ]; then
			echo "needs formatting: $file"
			status=1
		fi
	else
		clang-format -i "$file"
		sed -i -e :a -e '/^\n*$/{$d;N;ba' -e '}' "$file"
	fi
done < <(find core_scheduler_b200/csrc examples tests/cpp baseline -type f \
	-not \( -path '*/build/*' -o -path 'baseline/_ref/*' \) \
	\( -name '*.cpp' -o -name '*.h' -o -name '*.cu' -o -name '*.cuh' \) -print0)
if [ "${1:-}" != "--check" ]; then echo "All files have been formatted."; fi
exit $status
